// Vector-engine kernels for the "gcn" message pattern, value type float.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_gcn_f32, float, VOP_COPY_RHS, ROP_NOOP, VSC_NOOP, AOP_ADD)
}
