// fusedmm_inst.cuh -- stamps out the vector-engine kernels of ONE (value type, message pattern) pair.
// Each inst_*.cu includes this once, so the patterns compile in parallel.
#pragma once
#include "fusedmm_kernels.cuh"

namespace fmm {

// (lanes per edge G, 16-byte vectors per lane NV, gathers in flight per slot U).  G*NV*16 bytes is
// the longest row a tiling covers; U is sized so that a lane holds at most 8 gathered vectors.
#define FMM_FOR_EACH_TILING(X) \
   X(4, 1, 4) X(8, 1, 8) X(8, 2, 4) X(8, 4, 2) X(16, 1, 8) X(16, 2, 4) X(16, 4, 2) \
   X(32, 1, 8) X(32, 2, 4) X(32, 4, 2) X(32, 8, 1)

#define FMM_TILING_CASE(G_, NV_, U_)                                                                 \
   case ((G_) << 8) | (NV_):                                                                          \
      fused_vec_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_>                                   \
         <<<static_cast<unsigned int>(grid), WARPS_PER_CTA * 32, 0, stream>>>(p);                     \
      return true;

#define FMM_DEFINE_PATTERN_LAUNCHER(FN, T, VOPC, ROPC, VSCC, AOPC)                                   \
   bool FN(int G, int NV, const Params<T> &p, long long grid, cudaStream_t stream)                    \
   {                                                                                                  \
      using T_ = T;                                                                                   \
      constexpr int VOPC_ = VOPC, ROPC_ = ROPC, VSCC_ = VSCC, AOPC_ = AOPC;                           \
      switch ((G << 8) | NV) {                                                                        \
         FMM_FOR_EACH_TILING(FMM_TILING_CASE)                                                         \
         default: return false;                                                                       \
      }                                                                                               \
   }

}  // namespace fmm
