// Vector-engine kernels for the "generic" message pattern, value type float.
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_generic_f32, float, RT, RT, RT, RT)
}
