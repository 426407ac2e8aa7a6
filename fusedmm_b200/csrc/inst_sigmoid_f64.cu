// Vector-engine kernels for the "sigmoid" message pattern, value type double.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_sigmoid_f64, double, VOP_COPY_RHS, ROP_DOT, VSC_MUL, AOP_ADD)
}
