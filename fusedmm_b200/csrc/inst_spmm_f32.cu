// Vector-engine kernels for the "spmm" message pattern, value type float.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_spmm_f32, float, VOP_COPY_RHS, ROP_NOOP, VSC_MUL, AOP_ADD)
}
