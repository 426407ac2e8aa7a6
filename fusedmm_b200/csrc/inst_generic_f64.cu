// Vector-engine kernels for the "generic" message pattern, value type double.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_generic_f64, double, RT, RT, RT, RT)
}
