// Vector-engine kernels for the "generic" message pattern, value type double.
// the flag-interpreting (32, 2, 4) kernel is faster with an 80-register budget; the specialised ones are not
#define FMM_FOR_EACH_EXTRA_TILING(X) X(32, 2, 4, 3)
#include "fusedmm_inst.cuh"
namespace fmm {
FMM_DEFINE_PATTERN_LAUNCHER(launch_vec_generic_f64, double, RT, RT, RT, RT)
}
