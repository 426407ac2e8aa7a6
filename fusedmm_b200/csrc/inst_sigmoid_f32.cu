// Vector-engine kernels for the "sigmoid" message pattern, value type float.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_sigmoid_f32, float, VOP_COPY_RHS, ROP_DOT, VSC_MUL, AOP_ADD)
}
