// Vector-engine kernels for the "spmm" message pattern, value type double.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_spmm_f64, double, VOP_COPY_RHS, ROP_NOOP, VSC_MUL, AOP_ADD)
}
