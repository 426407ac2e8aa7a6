// fusedmm_inst.cuh -- stamps out the kernels of ONE (value type, message pattern) pair.
// Each inst_*.cu includes this once, so the patterns compile in parallel.
#pragma once
#include "fusedmm_kernels.cuh"
#include "fusedmm_stream.cuh"
#include "fusedmm_bulk.cuh"

namespace fmm {

// Row scheduler: (lanes per edge G, 16-byte vectors per lane NV, gathers in flight per slot U, register
// budget class MB).  G*NV*16 bytes is the longest row a tiling covers.
#define FMM_FOR_EACH_TILING(X) \
   X(4, 1, 4, 0) X(8, 1, 8, 0) X(8, 2, 4, 0) X(8, 4, 2, 0) X(16, 1, 8, 0) X(16, 2, 4, 0) X(16, 4, 2, 0) \
   X(32, 1, 8, 0) X(32, 2, 4, 0) X(32, 4, 2, 0) X(32, 8, 1, 0) X(32, 16, 1, 0) \
   X(16, 2, 8, 0) X(32, 2, 8, 0) X(8, 2, 4, 4) X(32, 4, 2, 3) X(16, 2, 4, 3) X(32, 2, 4, 3) X(16, 4, 2, 3)

// The default tilings once more for calls whose K fills the tiling exactly (K = G*NV*16 bytes: every power of two
// from 16 to 2048 floats, 8 to 1024 doubles): FLAG_EXACT_K drops the per-vector bounds predicates of every gather and
// store.  FR on R-MAT scale 20 at K = 256: 4.01 ms against 4.32; SpMM at K = 512: 27.8 against 28.6.  Two default
// tilings are left out because their exact forms measured slower: (16, 2, 8) for the chunks at K = 128 floats (R-MAT
// scale 24: chunk launch 30.5 ms against 25.8) and (8, 2, 4) at K = 64 floats (+1 %).
#define FMM_FOR_EACH_EXACT_TILING(X) \
   X(4, 1, 4, 0) X(8, 1, 8, 0) X(16, 2, 4, 3) X(32, 2, 4, 0) X(32, 2, 8, 0) X(32, 2, 4, 3) \
   X(32, 4, 2, 3) X(32, 8, 1, 0) X(32, 16, 1, 0) X(16, 4, 2, 3)

// The default tilings with one-element vectors (FLAG_ELEMENT), for calls whose K, leading dimensions or base addresses
// are not multiples of 16 bytes: K up to G*NV elements (512); 2-D / 3-D layouts (K = 2, 3) get 8 rows per warp.
#define FMM_FOR_EACH_ELEMENT_TILING(X) \
   X(4, 1, 4, 0) X(8, 1, 8, 0) X(8, 2, 4, 4) X(16, 2, 8, 0) X(32, 2, 4, 0) X(32, 4, 2, 3) X(32, 8, 1, 0) X(32, 16, 1, 0)

// 32-bit column ids (FLAG_OFFSET32: the address of a neighbour row in one multiply-add), plain and exact-K forms, for
// the one tiling that gains from it: whole rows of 17 to 32 vectors of 16 bytes (K = 128 floats on R-MAT scale 24: the
// call 40.4 -> 38.9 ms).  The 32-lane tilings lose with it in both launches although they execute fewer instructions
// (K = 128 doubles 80.4 -> 83.9 ms in the whole-row launch alone, 93.9 in both; K = 512 floats 23.4 -> 24.6 / 26.1;
// K = 256 floats 3.94 -> 4.10 / 4.13), and so does the chunk launch of K = 128 floats (24.0 -> 24.3 ms).
#define FMM_FOR_EACH_OFF32_TILING(X) X(16, 2, 4, 3)
#define FMM_FOR_EACH_OFF32_EXACT_TILING(X) X(16, 2, 4, 3)

// A translation unit may add tilings of its own by defining this before the include (the flag-interpreting
// kernels need other register budgets than the specialised ones).
#ifndef FMM_FOR_EACH_EXTRA_TILING
#define FMM_FOR_EACH_EXTRA_TILING(X)
#endif

// Edge-stream scheduler: (G, NV).
#define FMM_FOR_EACH_STREAM_TILING(X) \
   X(4, 1) X(8, 1) X(8, 2) X(8, 4) X(16, 1) X(16, 2) X(16, 4) X(32, 1) X(32, 2) X(32, 4) X(32, 8)

#define FMM_TILING_CASE(G_, NV_, U_, MB_)                                                            \
   case ((MB_) << 24) | ((U_) << 16) | ((G_) << 8) | (NV_):                                           \
      launch_kernel<T_>(fused_vec_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_, MB_>, grid,      \
                        warps * 32, stream, p);                                                       \
      return true;
#define FMM_ELEMENT_TILING_CASE(G_, NV_, U_, MB_)                                                    \
   case (2 << 28) | ((MB_) << 24) | ((U_) << 16) | ((G_) << 8) | (NV_):                               \
      launch_kernel<T_>(fused_vec_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_, MB_,             \
                                         FLAG_ELEMENT>, grid, warps * 32, stream, p);                 \
      return true;
#define FMM_EXACT_TILING_CASE(G_, NV_, U_, MB_)                                                      \
   case (1 << 28) | ((MB_) << 24) | ((U_) << 16) | ((G_) << 8) | (NV_):                               \
      launch_kernel<T_>(fused_vec_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_, MB_,             \
                                         FLAG_EXACT_K>, grid, warps * 32, stream, p);                 \
      return true;

#define FMM_OFF32_TILING_CASE(G_, NV_, U_, MB_)                                                      \
   case (4 << 28) | ((MB_) << 24) | ((U_) << 16) | ((G_) << 8) | (NV_):                               \
      launch_kernel<T_>(fused_vec_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_, MB_,             \
                                         FLAG_OFFSET32>, grid, warps * 32, stream, p);                \
      return true;
#define FMM_OFF32_EXACT_TILING_CASE(G_, NV_, U_, MB_)                                                \
   case (5 << 28) | ((MB_) << 24) | ((U_) << 16) | ((G_) << 8) | (NV_):                               \
      launch_kernel<T_>(fused_vec_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_, MB_,             \
                                         FLAG_OFFSET32 | FLAG_EXACT_K>, grid, warps * 32, stream, p); \
      return true;

// persistent launch of the edge-stream kernel: as many CTAs as fit on the device at once
#define FMM_STREAM_CASE(G_, NV_)                                                                     \
   case ((G_) << 8) | (NV_): {                                                                        \
      auto kern = fused_stream_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_>;                       \
      const size_t smem = static_cast<size_t>(warps) * p.depth * (NV_) * 512;                         \
      if (smem > 48 * 1024 &&                                                                         \
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                     \
                               static_cast<int>(smem)) != cudaSuccess) return false;                  \
      int per_sm = 0;                                                                                 \
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, warps * 32, smem)              \
             != cudaSuccess || per_sm < 1) return false;                                              \
      kern<<<static_cast<unsigned int>(sm_count * per_sm), warps * 32, smem, stream>>>(p);            \
      return true;                                                                                    \
   }

// Chunk launch through bulk copies (fusedmm_bulk.cuh): (G, NV, U, ring slots D).
#define FMM_FOR_EACH_BULK_TILING(X) \
   X(8, 2, 4, 16) X(8, 2, 4, 32) X(16, 2, 4, 16) X(16, 2, 4, 32) X(32, 2, 4, 16) X(32, 2, 4, 32) X(32, 4, 2, 16) X(32, 4, 2, 32)

// persistent launch: as many CTAs as fit at once (the ring of every warp lives in dynamic shared memory)
#define FMM_BULK_CASE(G_, NV_, U_, D_)                                                               \
   case ((D_) << 16) | ((G_) << 8) | (NV_): {                                                         \
      auto kern = fused_bulk_chunk_kernel<T_, VOPC_, ROPC_, VSCC_, AOPC_, G_, NV_, U_, D_, 0>;        \
      const size_t smem = static_cast<size_t>(warps) * (D_) * ((G_) * (NV_) * 16 + 8);                \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                     \
                               static_cast<int>(smem)) != cudaSuccess) { cudaGetLastError(); return false; } \
      int per_sm = 0;                                                                                 \
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, warps * 32, smem)              \
             != cudaSuccess || per_sm < 1) { cudaGetLastError(); return false; }                      \
      if (max_per_sm > 0 && per_sm > max_per_sm) per_sm = max_per_sm;                                 \
      return launch_kernel<T_>(kern, static_cast<long long>(sm_count) * per_sm, warps * 32, stream, p, smem) == cudaSuccess; \
   }

#define FMM_DEFINE_PATTERN_LAUNCHER(FN, T, VOPC, ROPC, VSCC, AOPC)                                   \
   bool FN##_bulk(int G, int NV, int D, int warps, const Params<T> &p, int sm_count, int max_per_sm,   \
                  cudaStream_t stream)                                                                \
   {                                                                                                  \
      using T_ = T;                                                                                   \
      constexpr int VOPC_ = VOPC, ROPC_ = ROPC, VSCC_ = VSCC, AOPC_ = AOPC;                           \
      if (VOPC_ < 0) return false; /* the flag-interpreting instantiation has no bulk form */         \
      switch ((D << 16) | (G << 8) | NV) {                                                            \
         FMM_FOR_EACH_BULK_TILING(FMM_BULK_CASE)                                                      \
         default: return false;                                                                       \
      }                                                                                               \
   }                                                                                                  \
   bool FN##_stream(int G, int NV, int warps, const Params<T> &p, int sm_count, cudaStream_t stream)  \
   {                                                                                                  \
      using T_ = T;                                                                                   \
      constexpr int VOPC_ = VOPC, ROPC_ = ROPC, VSCC_ = VSCC, AOPC_ = AOPC;                           \
      switch ((G << 8) | NV) {                                                                        \
         FMM_FOR_EACH_STREAM_TILING(FMM_STREAM_CASE)                                                  \
         default: return false;                                                                       \
      }                                                                                               \
   }                                                                                                  \
   bool FN(int G, int NV, int U, int warps, const Params<T> &p, long long grid, cudaStream_t stream)  \
   {                                                                                                  \
      using T_ = T;                                                                                   \
      constexpr int VOPC_ = VOPC, ROPC_ = ROPC, VSCC_ = VSCC, AOPC_ = AOPC;                           \
      /* U carries the register budget class MB in bits 8..15 (0 = compiler's choice) and the call-shape   */ \
      /* flags in bits 16..: 1 = FLAG_EXACT_K, 2 = FLAG_ELEMENT (never both here), 4 = FLAG_OFFSET32       */ \
      const int MB = (U >> 8) & 0xFF, FL = (U >> 16) & 7;                                             \
      U &= 0xFF;                                                                                      \
      switch ((FL << 28) | (MB << 24) | (U << 16) | (G << 8) | NV) {                                  \
         FMM_FOR_EACH_TILING(FMM_TILING_CASE)                                                         \
         FMM_FOR_EACH_EXTRA_TILING(FMM_TILING_CASE)                                                   \
         FMM_FOR_EACH_EXACT_TILING(FMM_EXACT_TILING_CASE)                                             \
         FMM_FOR_EACH_ELEMENT_TILING(FMM_ELEMENT_TILING_CASE)                                         \
         FMM_FOR_EACH_OFF32_TILING(FMM_OFF32_TILING_CASE)                                             \
         FMM_FOR_EACH_OFF32_EXACT_TILING(FMM_OFF32_EXACT_TILING_CASE)                                 \
         default: return false;                                                                       \
      }                                                                                               \
   }

}  // namespace fmm
