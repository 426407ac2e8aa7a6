// Vector-engine kernels for the "tdist" message pattern, value type double.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_tdist_f64, double, VOP_SUBR, ROP_NORMR, VSC_MUL, AOP_ADD)
}
