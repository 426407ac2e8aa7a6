// Vector-engine kernels for the "tdist" message pattern, value type float.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_tdist_f32, float, VOP_SUBR, ROP_NORMR, VSC_MUL, AOP_ADD)
}
