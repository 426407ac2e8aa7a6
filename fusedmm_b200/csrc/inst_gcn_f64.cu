// Vector-engine kernels for the "gcn" message pattern, value type double.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_gcn_f64, double, VOP_COPY_RHS, ROP_NOOP, VSC_NOOP, AOP_ADD)
}
