// fusedmm_capi.cu -- the C ABI of libfusedmm_b200.so (include/fusedmm_b200.h): message decoding,
// SOP resolution, pointer residency and staging, the host half of the row scheduler, kernel dispatch.
//
// Mirrors the control flow of the reference's entry point (HipGraph/FusedMM fusedMM.c:487-744):
// recognise the four optimised message patterns first (:512-605), otherwise validate each stage code
// in the reference's order and run the flag-interpreting path (:610-739).  There is no CPU path: if
// CUDA is unusable the call fails with FUSEDMM_B200_ERR_CUDA.
#include "../../include/fusedmm_b200.h"
#include "fusedmm_kernels.cuh"
#include "fusedmm_stream.cuh"

#include <nvtx3/nvToolsExt.h>  // header-only: the ranges cost nothing unless a profiler is attached

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

// The inspector's result (fusedmm_b200_plan_create): the CSR resident on one device and its split-row list.
struct fusedmm_b200_plan {
   int device = -1;
   int ptr_bits = 64, idx_bits = 32, val_dtype = -1;  // val_dtype: -1 no values, 0 float, 1 double
   long long m = 0, nnz = 0, chunk = 512;
   void *own[4] = {nullptr, nullptr, nullptr, nullptr};  // device copies made from host arrays (val, indx, pntrb, pntre)
   const void *val = nullptr, *indx = nullptr, *pntrb = nullptr, *pntre = nullptr;  // device addresses used by the calls
   long long *hub_row = nullptr, *hub_base = nullptr;
   long long *order = nullptr;             // visiting order of the chunks (sorted by first column id), or null
   unsigned int *row_order = nullptr;      // whole rows sorted by length inside windows, or null
   unsigned long long *counter = nullptr;  // packed (split rows << HUB_SHIFT) | chunks, written once by the scan
   long long nh = 0, nchunks = 0;
};

namespace fmm {

// per-pattern launchers (inst_*.cu)
#define FMM_DECLARE_LAUNCHER(PN)                                                                      \
   bool launch_vec_##PN##_f32(int, int, int, int, const Params<float> &, long long, cudaStream_t);    \
   bool launch_vec_##PN##_f64(int, int, int, int, const Params<double> &, long long, cudaStream_t);   \
   bool launch_vec_##PN##_f32_stream(int, int, int, const Params<float> &, int, cudaStream_t);        \
   bool launch_vec_##PN##_f64_stream(int, int, int, const Params<double> &, int, cudaStream_t);       \
   bool launch_vec_##PN##_f32_bulk(int, int, int, int, const Params<float> &, int, int, cudaStream_t); \
   bool launch_vec_##PN##_f64_bulk(int, int, int, int, const Params<double> &, int, int, cudaStream_t);
FMM_DECLARE_LAUNCHER(generic)
FMM_DECLARE_LAUNCHER(sigmoid)
FMM_DECLARE_LAUNCHER(tdist)
FMM_DECLARE_LAUNCHER(spmm)
FMM_DECLARE_LAUNCHER(gcn)

template <>
bool launch_vec<float>(int pattern, int G, int NV, int U, int warps, const Params<float> &p, long long grid, cudaStream_t s)
{
   switch (pattern) {
      case PAT_SIGMOID: return launch_vec_sigmoid_f32(G, NV, U, warps, p, grid, s);
      case PAT_TDIST:   return launch_vec_tdist_f32(G, NV, U, warps, p, grid, s);
      case PAT_SPMM:    return launch_vec_spmm_f32(G, NV, U, warps, p, grid, s);
      case PAT_GCN:     return launch_vec_gcn_f32(G, NV, U, warps, p, grid, s);
      default:          return launch_vec_generic_f32(G, NV, U, warps, p, grid, s);
   }
}
template <>
bool launch_vec<double>(int pattern, int G, int NV, int U, int warps, const Params<double> &p, long long grid, cudaStream_t s)
{
   switch (pattern) {
      case PAT_SIGMOID: return launch_vec_sigmoid_f64(G, NV, U, warps, p, grid, s);
      case PAT_TDIST:   return launch_vec_tdist_f64(G, NV, U, warps, p, grid, s);
      case PAT_SPMM:    return launch_vec_spmm_f64(G, NV, U, warps, p, grid, s);
      case PAT_GCN:     return launch_vec_gcn_f64(G, NV, U, warps, p, grid, s);
      default:          return launch_vec_generic_f64(G, NV, U, warps, p, grid, s);
   }
}
template <typename T>
bool launch_bulk(int pattern, int G, int NV, int D, int warps, const Params<T> &p, int sm_count, int max_per_sm, cudaStream_t s);
template <>
bool launch_bulk<float>(int pattern, int G, int NV, int D, int warps, const Params<float> &p, int sm_count, int max_per_sm, cudaStream_t s)
{
   switch (pattern) {
      case PAT_SIGMOID: return launch_vec_sigmoid_f32_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      case PAT_TDIST:   return launch_vec_tdist_f32_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      case PAT_SPMM:    return launch_vec_spmm_f32_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      case PAT_GCN:     return launch_vec_gcn_f32_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      default:          return false;
   }
}
template <>
bool launch_bulk<double>(int pattern, int G, int NV, int D, int warps, const Params<double> &p, int sm_count, int max_per_sm, cudaStream_t s)
{
   switch (pattern) {
      case PAT_SIGMOID: return launch_vec_sigmoid_f64_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      case PAT_TDIST:   return launch_vec_tdist_f64_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      case PAT_SPMM:    return launch_vec_spmm_f64_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      case PAT_GCN:     return launch_vec_gcn_f64_bulk(G, NV, D, warps, p, sm_count, max_per_sm, s);
      default:          return false;
   }
}
template <typename T>
bool launch_stream(int pattern, int G, int NV, int warps, const Params<T> &p, int sm_count, cudaStream_t s);
template <>
bool launch_stream<float>(int pattern, int G, int NV, int warps, const Params<float> &p, int sm_count, cudaStream_t s)
{
   switch (pattern) {
      case PAT_SIGMOID: return launch_vec_sigmoid_f32_stream(G, NV, warps, p, sm_count, s);
      case PAT_TDIST:   return launch_vec_tdist_f32_stream(G, NV, warps, p, sm_count, s);
      case PAT_SPMM:    return launch_vec_spmm_f32_stream(G, NV, warps, p, sm_count, s);
      case PAT_GCN:     return launch_vec_gcn_f32_stream(G, NV, warps, p, sm_count, s);
      default:          return launch_vec_generic_f32_stream(G, NV, warps, p, sm_count, s);
   }
}
template <>
bool launch_stream<double>(int pattern, int G, int NV, int warps, const Params<double> &p, int sm_count, cudaStream_t s)
{
   switch (pattern) {
      case PAT_SIGMOID: return launch_vec_sigmoid_f64_stream(G, NV, warps, p, sm_count, s);
      case PAT_TDIST:   return launch_vec_tdist_f64_stream(G, NV, warps, p, sm_count, s);
      case PAT_SPMM:    return launch_vec_spmm_f64_stream(G, NV, warps, p, sm_count, s);
      case PAT_GCN:     return launch_vec_gcn_f64_stream(G, NV, warps, p, sm_count, s);
      default:          return launch_vec_generic_f64_stream(G, NV, warps, p, sm_count, s);
   }
}
template <typename T>
void launch_any(const Params<T> &p, int warps, long long grid, cudaStream_t s)
{
   launch_kernel<T>(fused_any_kernel<T>, grid, warps * 32, s, p, static_cast<size_t>(warps) * ANY_MAX_CACHED * sizeof(T));
}
template <typename T>
void launch_fixup(const Params<T> &p, long long grid, cudaStream_t s)
{
   launch_kernel<T>(hub_fixup_kernel<T>, grid, WARPS_PER_CTA * 32, s, p);
}

__global__ void scan_hub_rows(const void *pntrb, const void *pntre, int ptr64, long long m,
                              long long chunk, unsigned long long *counter, long long *hub_row,
                              long long *hub_base, long long hub_cap)
{
   grid_launch_dependents();  // the chunk launch that follows may become resident while this scan runs
   const long long r = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
   if (r >= m) return;
   const long long deg = ld_index(pntre, r, ptr64) - ld_index(pntrb, r, ptr64);
   if (deg > chunk) {
      const unsigned long long nch = static_cast<unsigned long long>((deg + chunk - 1) / chunk);
      const unsigned long long old = atomicAdd(counter, (1ull << HUB_SHIFT) + nch);
      const long long slot = static_cast<long long>(old >> HUB_SHIFT);
      if (slot < hub_cap) {
         hub_row[slot] = r;
         hub_base[slot] = static_cast<long long>(old & HUB_CHUNK_MASK);
      }
   }
}

// ---- order of the whole rows (option row_bins) --------------------------------------------------------
// The whole-row launch gives every group of G lanes of a warp its own row and the 32/G rows of a warp run in
// lockstep, so a warp takes as long as its longest row.  On a skewed graph neighbouring rows differ widely (R-MAT
// scale 20: 58 % of the slot-iterations do work; with rows of equal length side by side, 91 %).  This kernel sorts
// the rows of every window of ROW_BIN_TILE consecutive rows by their number of edges, longest first (a counting sort
// in shared memory), and writes the permutation; rows without edges and split rows (which the whole-row launch
// skips) come last.  Rows stay inside their window, so X, Z and the row pointers are still read window by window.
constexpr int ROW_BIN_TILE = 2048, ROW_BIN_KEYS = 258;

__global__ void __launch_bounds__(256)
bin_rows_kernel(const void *pntrb, const void *pntre, int ptr64, long long m, long long chunk, unsigned int *row_order)
{
   __shared__ unsigned int hist[ROW_BIN_KEYS];
   constexpr int PER = ROW_BIN_TILE / 256;
   const long long base = static_cast<long long>(blockIdx.x) * ROW_BIN_TILE;
   for (int b = threadIdx.x; b < ROW_BIN_KEYS; b += 256) hist[b] = 0;
   __syncthreads();
   int key[PER];
#pragma unroll
   for (int i = 0; i < PER; i++) {
      const long long r = base + i * 256 + threadIdx.x;
      key[i] = -1;
      if (r < m) {
         const long long deg = ld_index(pntre, r, ptr64) - ld_index(pntrb, r, ptr64);
         // bin 0: the longest whole rows ... bin 256: one edge; bin 257: nothing to do in the whole-row launch
         key[i] = (deg <= 0 || deg > chunk) ? ROW_BIN_KEYS - 1 : (deg >= 256 ? 0 : 256 - static_cast<int>(deg));
         atomicAdd(hist + key[i], 1u);
      }
   }
   __syncthreads();
   if (threadIdx.x < 32) {  // exclusive prefix sums of the 258 counters by one warp
      unsigned int run = 0;
      for (int b0 = 0; b0 < ROW_BIN_KEYS; b0 += 32) {
         const int b = b0 + threadIdx.x;
         const unsigned int v = b < ROW_BIN_KEYS ? hist[b] : 0u;
         unsigned int inc = v;
         for (int off = 1; off < 32; off <<= 1) {
            const unsigned int up = __shfl_up_sync(FULL, inc, off);
            if (static_cast<int>(threadIdx.x) >= off) inc += up;
         }
         if (b < ROW_BIN_KEYS) hist[b] = run + inc - v;
         run += __shfl_sync(FULL, inc, 31);
      }
   }
   __syncthreads();
#pragma unroll
   for (int i = 0; i < PER; i++)
      if (key[i] >= 0) row_order[base + atomicAdd(hist + key[i], 1u)] = static_cast<unsigned int>(base + i * 256 + threadIdx.x);
}

// ---- visiting order of the chunks of split rows (option chunk_order) ---------------------------------
// Counting sort of the chunks by the column id of their first edge, scaled to ORDER_BUCKETS buckets: count, prefix
// sums, placement.  The order inside a bucket is whatever the atomics give; results do not depend on it (every chunk
// writes its own partial sum and the fix-up adds them in chunk order).
constexpr int ORDER_BUCKETS = 4096;

__device__ __forceinline__ int order_bucket(const void *indx, int idx64, long long e, long long ncols)
{
   const long long col = ld_index(indx, e, idx64);
   long long b = ncols > 0 ? static_cast<long long>((static_cast<unsigned long long>(col < 0 ? 0 : col) * ORDER_BUCKETS) / static_cast<unsigned long long>(ncols)) : 0;
   return static_cast<int>(b < ORDER_BUCKETS ? b : ORDER_BUCKETS - 1);
}

// pass = 0: cnt[bucket] += chunks of that bucket; pass = 1: the chunks are written into order[] at off[bucket] onward;
// pass = 2: *(unsigned long long *)cnt = max(first column id of a chunk) + 1 (a stand-in for the column count).
// One warp per split row.  A block counts its chunks in a shared-memory histogram first, so that the global counters
// see one addition per block and bucket (the first chunk of nearly every row of a skewed graph falls into bucket 0);
// for the placement the block reserves its part of every bucket with that one addition and then hands out positions
// from shared memory.
__global__ void __launch_bounds__(256)
order_chunks_kernel(int pass, const void *pntrb, const void *pntre, int ptr64, const void *indx, int idx64,
                    long long ncols, long long chunk, const unsigned long long *counter,
                    const long long *hub_row, const long long *hub_base, long long hub_cap,
                    long long chunk_cap, unsigned int *cnt, const unsigned int *off, long long *order)
{
   __shared__ unsigned int h[ORDER_BUCKETS];
   const unsigned long long c = *counter;
   const long long nh = static_cast<long long>(c >> HUB_SHIFT), nchunks = static_cast<long long>(c & HUB_CHUNK_MASK);
   if (nh > hub_cap || nchunks > chunk_cap) return;
   const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
   const long long first = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5);
   const long long stride = static_cast<long long>(gridDim.x) * wpb;
   if (first - (threadIdx.x >> 5) >= nh) return;  // no split row for this block
   if (pass == 2) {
      unsigned long long *top = reinterpret_cast<unsigned long long *>(cnt);
      unsigned long long mine = 0;
      for (long long slot = first; slot < nh; slot += stride) {
         const long long row = hub_row[slot];
         const long long eb = ld_index(pntrb, row, ptr64), ee = ld_index(pntre, row, ptr64);
         const long long nc = (ee - eb + chunk - 1) / chunk;
         for (long long q = lane; q < nc; q += 32) {
            const long long col = ld_index(indx, eb + q * chunk, idx64);
            if (col >= 0 && static_cast<unsigned long long>(col) + 1 > mine) mine = static_cast<unsigned long long>(col) + 1;
         }
      }
      if (mine > *reinterpret_cast<volatile unsigned long long *>(top)) atomicMax(top, mine);
      return;
   }
   for (int b = threadIdx.x; b < ORDER_BUCKETS; b += blockDim.x) h[b] = 0;
   __syncthreads();
   for (int round = 0; round <= pass; round++) {
      for (long long slot = first; slot < nh; slot += stride) {
         const long long row = hub_row[slot], base = hub_base[slot];
         const long long eb = ld_index(pntrb, row, ptr64), ee = ld_index(pntre, row, ptr64);
         const long long nc = (ee - eb + chunk - 1) / chunk;
         for (long long q = lane; q < nc; q += 32) {
            const int b = order_bucket(indx, idx64, eb + q * chunk, ncols);
            const unsigned int at = atomicAdd(h + b, 1u);
            if (round == 1) order[at] = base + q;
         }
      }
      __syncthreads();
      if (round == 0) {
         for (int b = threadIdx.x; b < ORDER_BUCKETS; b += blockDim.x) {
            const unsigned int mine = h[b];
            if (pass == 0) { if (mine) atomicAdd(cnt + b, mine); }
            else h[b] = mine ? off[b] + atomicAdd(cnt + b, mine) : 0u;  // from here on: the next position of the bucket
         }
         __syncthreads();
      }
   }
}

__global__ void order_scan_kernel(const unsigned int *cnt, unsigned int *off);

// The three launches of the sort.  cnt: 3 x ORDER_BUCKETS counters (counts, offsets, fill marks).
static cudaError_t enqueue_chunk_order(const void *pntrb, const void *pntre, int ptr64, const void *indx, int idx64, long long ncols,
                                       long long chunk, const unsigned long long *counter, const long long *hub_row,
                                       const long long *hub_base, long long hub_cap, long long chunk_cap, unsigned int *cnt,
                                       long long *order, int sm_count, cudaStream_t s)
{
   const unsigned int grid = static_cast<unsigned int>(sm_count * 8);
   cudaError_t e = cudaMemsetAsync(cnt, 0, 3 * ORDER_BUCKETS * sizeof(unsigned int), s);
   if (e != cudaSuccess) return e;
   order_chunks_kernel<<<grid, 256, 0, s>>>(0, pntrb, pntre, ptr64, indx, idx64, ncols, chunk, counter, hub_row, hub_base, hub_cap,
                                            chunk_cap, cnt, nullptr, nullptr);
   order_scan_kernel<<<1, 1024, 0, s>>>(cnt, cnt + ORDER_BUCKETS);
   order_chunks_kernel<<<grid, 256, 0, s>>>(1, pntrb, pntre, ptr64, indx, idx64, ncols, chunk, counter, hub_row, hub_base, hub_cap,
                                            chunk_cap, cnt + 2 * ORDER_BUCKETS, cnt + ORDER_BUCKETS, order);
   return cudaGetLastError();
}

// off[b] = cnt[0] + ... + cnt[b-1]; one block of 1024 threads, four buckets per thread
__global__ void order_scan_kernel(const unsigned int *cnt, unsigned int *off)
{
   __shared__ unsigned int sums[1024];
   constexpr int PER = ORDER_BUCKETS / 1024;
   unsigned int v[PER], s = 0;
   for (int i = 0; i < PER; i++) { v[i] = cnt[threadIdx.x * PER + i]; s += v[i]; }
   sums[threadIdx.x] = s;
   __syncthreads();
   for (int d = 1; d < 1024; d <<= 1) {
      const unsigned int add = threadIdx.x >= d ? sums[threadIdx.x - d] : 0u;
      __syncthreads();
      sums[threadIdx.x] += add;
      __syncthreads();
   }
   unsigned int run = sums[threadIdx.x] - s;
   for (int i = 0; i < PER; i++) { off[threadIdx.x * PER + i] = run; run += v[i]; }
}

// Validation of a CSR: counts rows whose end precedes their start, column ids outside [0, n), edges, and
// the largest degree.  report[0..3] must be zero on entry.
__global__ void check_csr_kernel(const void *pntrb, const void *pntre, const void *indx, int ptr64, int idx64,
                                 long long m, long long n, unsigned long long *report)
{
   const int lane = threadIdx.x & 31;
   const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
   unsigned long long bad_rows = 0, bad_cols = 0, edges = 0, maxdeg = 0;
   for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < m; r += nwarps) {
      const long long b = ld_index(pntrb, r, ptr64), e = ld_index(pntre, r, ptr64);
      if (e < b || b < 0) { if (lane == 0) bad_rows++; continue; }
      if (lane == 0) { edges += static_cast<unsigned long long>(e - b); maxdeg = max(maxdeg, static_cast<unsigned long long>(e - b)); }
      for (long long j = b + lane; j < e; j += 32) {
         const long long c = ld_index(indx, j, idx64);
         if (c < 0 || c >= n) bad_cols++;
      }
   }
   if (bad_rows) atomicAdd(report + 0, bad_rows);
   if (bad_cols) atomicAdd(report + 1, bad_cols);
   if (edges) atomicAdd(report + 2, edges);
   if (maxdeg) atomicMax(report + 3, maxdeg);
}

}  // namespace fmm

namespace {

using namespace fmm;

// ---------------------------------------------------------------------------------------------------
// process-wide state
// ---------------------------------------------------------------------------------------------------
struct DevBuf {
   void *ptr = nullptr;
   size_t bytes = 0;
};

struct DeviceCtx {
   std::mutex mu;  // one call at a time per device; calls on different devices (from different host threads) overlap
   int device = -1;
   bool ready = false;
   cudaStream_t stream = nullptr;
   cudaEvent_t ev0 = nullptr, ev1 = nullptr;
   cudaEvent_t evk[4] = {nullptr, nullptr, nullptr, nullptr};  // after scan / rows; start and end of the chunk launch
   cudaStream_t side = nullptr;                 // the chunk and fix-up launches run beside the whole-row launch
   // the same at the device's greatest stream priority (option side_priority, the default): when both launches are
   // pending the block scheduler then places the chunk CTAs of split rows first, which measured 3-8 % faster
   cudaStream_t side_hi = nullptr;
   cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_side_end = nullptr;
   cudaStream_t copy = nullptr;                 // copies finished blocks of Z back to the host while later blocks compute
   cudaEvent_t ev_block[8] = {};
   // brings the column ids / edge values of the later blocks of such a call to the device while earlier blocks compute
   // and go back (the two directions of the link at once)
   cudaStream_t copy_in = nullptr;
   cudaEvent_t ev_in[8] = {}, ev_inputs = nullptr;
   int sm_count = 148;
   DevBuf stage[7];  // val, indx, pntrb, pntre, x, y, z
   DevBuf counter, hub_row, hub_base, partials;
   DevBuf row_order;  // option row_bins: permutation of the rows for the whole-row launch
   DevBuf order, order_cnt;  // option chunk_order: visiting order of the chunks; 3 x ORDER_BUCKETS counters
   long long hub_cap = 0;
   DevBuf part, heads;       // edge-stream scheduler scratch
   long long part_cap = 0;   // quanta the partition array has room for
   int async_engine = 0;     // engine of the latest asynchronous call (1 whole rows, 2 edge stream)
   long long async_quantum = 0;
   DevBuf table_f, table_d;
   // bookkeeping of the latest asynchronous call, for fusedmm_b200_stream_status
   bool async_pending = false;
   long long async_k = 0;
   size_t async_elt = 4;
};

struct Options {
   int64_t beta_mode = 0, accept_vop_noop = 0, hub_chunk = 256, force_tiling = 0, force_generic = 0, warps_per_cta = 1,
           engine = 0, edge_quantum = 256, stream_depth = 16, side_priority = 1, chunk_ctas_per_sm = 3, chunk_order = 1, row_bins = 1, blocked_inputs = 1, side_stream = 1, force_tiling_rows = 0,
           strict_udef = 0, multi_skip_empty_rows = 1, jit = 1, pdl = 1, timing_detail = 1, jit_call_shape = 0, jit_shape_mask = 3, offset32 = 1, exact_k = 1, element_vectors = 1, bulk_chunks = 0, bulk_warps = 8, bulk_ctas_per_sm = 0, hub_cap_initial = 1 << 16;
};

// Locking: g_mu guards the process-wide settings (options, default SOP) and the creation of device contexts; each
// device context has its own mutex for the body of a call.  A call copies the options into t_opt under g_mu and works
// on that copy, so host threads that drive different GPUs run their calls side by side.
constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
DeviceCtx g_ctx[MAX_DEVICES];
Options g_opt;
thread_local Options t_opt;
fusedmm_b200_sop g_sop = {FUSEDMM_SOP_SIGMOID, 0, 0.0, 0.0, 0.0};
thread_local fusedmm_b200_call_info t_info = {};

// An NVTX range that closes when the scope is left (whatever return path is taken).
struct NvtxRange {
   explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
   ~NvtxRange() { nvtxRangePop(); }
};

#define CK(call)                                                                                      \
   do {                                                                                               \
      cudaError_t e_ = (call);                                                                        \
      if (e_ != cudaSuccess) {                                                                        \
         fprintf(stderr, "fusedmm_b200: %s failed: %s (%s:%d)\n", #call, cudaGetErrorString(e_),      \
                 __FILE__, __LINE__);                                                                 \
         return e_ == cudaErrorMemoryAllocation ? FUSEDMM_B200_ERR_NOMEM : FUSEDMM_B200_ERR_CUDA;     \
      }                                                                                               \
   } while (0)

#define CKI(call)                                                                                     \
   do {                                                                                               \
      int s_ = (call);                                                                                \
      if (s_ != 0) return s_;                                                                         \
   } while (0)

int64_t g_fail_alloc_in = 0;  // option "inject_alloc_failure": the n-th device allocation from now on fails

int ensure_buf(DevBuf &b, size_t bytes)
{
   if (b.bytes >= bytes && b.ptr) return 0;
   if (g_fail_alloc_in > 0 && --g_fail_alloc_in == 0) {
      fprintf(stderr, "fusedmm_b200: injected allocation failure (%zu bytes)\n", bytes);
      return FUSEDMM_B200_ERR_NOMEM;
   }
   if (b.ptr) CK(cudaFree(b.ptr));
   b.ptr = nullptr;
   b.bytes = 0;
   // grow geometrically so that a sequence of slightly larger calls does not reallocate every time
   size_t want = std::max(bytes, static_cast<size_t>(256));
   CK(cudaMalloc(&b.ptr, want));
   b.bytes = want;
   return 0;
}

// Caller holds g_mu.
int get_ctx(DeviceCtx **out)
{
   int dev = 0;
   CK(cudaGetDevice(&dev));
   if (dev < 0 || dev >= MAX_DEVICES) return FUSEDMM_B200_ERR_LIMIT;
   DeviceCtx &c = g_ctx[dev];
   if (!c.ready) {
      c.device = dev;
      CK(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
      CK(cudaEventCreate(&c.ev0));
      CK(cudaEventCreate(&c.ev1));
      for (auto &e : c.evk) CK(cudaEventCreate(&e));
      CK(cudaStreamCreateWithFlags(&c.side, cudaStreamNonBlocking));
      {
         int least = 0, greatest = 0;
         CK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
         CK(cudaStreamCreateWithPriority(&c.side_hi, cudaStreamNonBlocking, greatest));
      }
      CK(cudaEventCreateWithFlags(&c.ev_fork, cudaEventDisableTiming));
      CK(cudaEventCreateWithFlags(&c.ev_join, cudaEventDisableTiming));
      CK(cudaEventCreate(&c.ev_side_end));
      CK(cudaStreamCreateWithFlags(&c.copy, cudaStreamNonBlocking));
      for (auto &e : c.ev_block) CK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      CK(cudaStreamCreateWithFlags(&c.copy_in, cudaStreamNonBlocking));
      for (auto &e : c.ev_in) CK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      CK(cudaEventCreateWithFlags(&c.ev_inputs, cudaEventDisableTiming));
      CK(cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev));
      CKI(ensure_buf(c.counter, 256));
      CK(cudaMemset(c.counter.ptr, 0, 256));
      c.ready = true;
   }
   *out = &c;
   return 0;
}

// Snapshot of the settings + the current device's context, then that device's lock (held until `lk` dies).
int enter_device(DeviceCtx **c, std::unique_lock<std::mutex> *lk, fusedmm_b200_sop *default_sop = nullptr)
{
   {
      std::lock_guard<std::mutex> lock(g_mu);
      t_opt = g_opt;
      if (default_sop) *default_sop = g_sop;
      CKI(get_ctx(c));
   }
   *lk = std::unique_lock<std::mutex>((*c)->mu);
   return 0;
}

// ---------------------------------------------------------------------------------------------------
// scalar functions on the host: used only to recognise a caller's SOP_UDEF_FUNC, never to compute Z
// ---------------------------------------------------------------------------------------------------
template <typename T>
void build_sigmoid_table(std::vector<T> &t)
{
   // init_SM_TABLE, kernels/codegen/genheader.base:43-52 (x is rounded to the value type first)
   t.resize(SM_TABLE_SIZE);
   for (int i = 0; i < SM_TABLE_SIZE; i++) {
      T x = static_cast<T>(2.0 * 5.0 * i / SM_TABLE_SIZE - 5.0);
      t[i] = static_cast<T>(1.0 / (1 + std::exp(-static_cast<double>(x))));
   }
}

template <typename T>
T host_sop(T s, const fusedmm_b200_sop &k, const std::vector<T> &table)
{
   switch (k.kind) {
      case FUSEDMM_SOP_SIGMOID: return static_cast<T>(1.0 / (1.0 + std::exp(-static_cast<double>(s))));
      case FUSEDMM_SOP_SIGMOID_TABLE_C: {
         T sm;
         if (s > 5.0) sm = 1;
         else if (s < -5.0) sm = 0;
         else {
            int idx = static_cast<int>((static_cast<double>(s) + 5.0) * SM_TABLE_SIZE / (2.0 * 5.0));
            sm = table[std::min(idx, SM_TABLE_SIZE - 1)];
         }
         return static_cast<T>(1.0 - sm);
      }
      case FUSEDMM_SOP_FR: return static_cast<T>(1.0 + 1.0 / s);
      case FUSEDMM_SOP_TDIST: return static_cast<T>(1.0 / (1.0 + s));
      case FUSEDMM_SOP_TDIST_CLAMPED: {
         T v = static_cast<T>(-2.0 / (1.0 + s));
         return v > 5.0 ? T(5) : (v < -5.0 ? T(-5) : v);
      }
      case FUSEDMM_SOP_LL: return static_cast<T>(std::log2(1 + std::sqrt(static_cast<double>(s))));
      case FUSEDMM_SOP_FA: return static_cast<T>(std::sqrt(static_cast<double>(s)) + 1.0 / s);
      case FUSEDMM_SOP_AFFINE_RECIP: {
         T v = static_cast<T>(k.p0 / (k.p1 + s));
         if (k.p2 > 0) v = v > k.p2 ? static_cast<T>(k.p2) : (v < -k.p2 ? static_cast<T>(-k.p2) : v);
         return v;
      }
      default: return s;
   }
}

template <typename T>
bool close_enough(T a, T b)
{
   if (std::isnan(a) || std::isnan(b)) return std::isnan(a) && std::isnan(b);
   if (std::isinf(a) || std::isinf(b)) return a == b;
   const double tol = sizeof(T) == 4 ? 2e-6 : 1e-13;
   return std::fabs(static_cast<double>(a) - static_cast<double>(b)) <=
          tol * std::max(1.0, std::max(std::fabs(static_cast<double>(a)), std::fabs(static_cast<double>(b))));
}

// Evaluate the caller's host function at fixed points and find the built-in it equals.
template <typename T>
bool identify_udef(int (*hook)(T, T *), fusedmm_b200_sop *found)
{
   // inside and outside the table range of the tester's sigmoid (+-5), on both sides of its edges and of the
   // clamp of its t-distribution scale, at 0 and at large magnitudes: a function that agrees with a built-in
   // only on a middle range is not taken for it
   static const double pts[] = {-1000.0, -30.0, -8.5, -7.5, -5.0625, -4.96875, -3.0, -1.25, -0.625, -0.5, -0.0625, 0.0,
                                0.03125, 0.3, 0.75, 1.0, 1.7, 2.9, 4.2, 4.96875, 5.0625, 6.0, 11.0, 30.0, 1000.0};
   constexpr int NP = sizeof(pts) / sizeof(pts[0]);
   T got[NP];
   for (int i = 0; i < NP; i++) {
      got[i] = T(0);
      hook(static_cast<T>(pts[i]), &got[i]);
   }
   std::vector<T> table;
   build_sigmoid_table(table);
   static const int order[] = {FUSEDMM_SOP_SIGMOID, FUSEDMM_SOP_SIGMOID_TABLE_C, FUSEDMM_SOP_FR, FUSEDMM_SOP_TDIST,
                               FUSEDMM_SOP_TDIST_CLAMPED, FUSEDMM_SOP_LL, FUSEDMM_SOP_FA, FUSEDMM_SOP_IDENTITY};
   for (int kind : order) {
      fusedmm_b200_sop k = {kind, 0, 0.0, 0.0, 0.0};
      bool all = true;
      for (int i = 0; i < NP && all; i++) all = close_enough(got[i], host_sop(static_cast<T>(pts[i]), k, table));
      if (all) { *found = k; return true; }
   }
   // p0/(p1+s), optionally clamped to +-p2: solve from two points of the unclamped range
   const int ia = 15, ib = 17;  // s = 1.0 and s = 2.9
   const double oa = got[ia], ob = got[ib], sa = pts[ia], sb = pts[ib];
   if (std::isfinite(oa) && std::isfinite(ob) && oa != ob) {
      const double p1 = (ob * sb - oa * sa) / (oa - ob);
      const double p0 = oa * (p1 + sa);
      double vmax = 0;
      for (int i = 0; i < NP; i++) if (std::isfinite(static_cast<double>(got[i]))) vmax = std::max(vmax, std::fabs(static_cast<double>(got[i])));
      for (double clampv : {0.0, vmax}) {
         fusedmm_b200_sop k = {FUSEDMM_SOP_AFFINE_RECIP, 0, p0, p1, clampv};
         bool all = true;
         for (int i = 0; i < NP && all; i++) {
            T want = host_sop(static_cast<T>(pts[i]), k, table);
            const double tol = sizeof(T) == 4 ? 1e-5 : 1e-11;
            if (std::isfinite(static_cast<double>(want)) && std::isfinite(static_cast<double>(got[i])))
               all = std::fabs(static_cast<double>(want) - got[i]) <= tol * std::max(1.0, std::fabs(static_cast<double>(want)));
            else
               all = close_enough(got[i], want);
         }
         if (all) { *found = k; return true; }
      }
   }
   return false;
}

// ---------------------------------------------------------------------------------------------------
// message decoding
// ---------------------------------------------------------------------------------------------------
struct Decoded {
   int vop, rop, sop, vsc, aop;
   int pattern;  // PAT_*
};

// Validation order and codes of fusedMM.c:610-628; UDEF stages other than SOP have no device body
// and give the status their default stubs return (fusedMM_internal.h:50-84).
int decode_message(int32_t imessage, const Options &opt, Decoded *d)
{
   d->vop = imessage & 0xF;
   d->rop = (imessage >> 4) & 0xF;
   d->sop = (imessage >> 8) & 0xF;
   d->vsc = (imessage >> 12) & 0xF;
   d->aop = (imessage >> 16) & 0xF;
   const bool vop_ok = (d->vop >= 1 && d->vop <= 7) || d->vop == OP_UDEF || (d->vop == 0 && opt.accept_vop_noop);
   if (!vop_ok) { fprintf(stderr, "Unknown VOP Message\n"); return FUSEDMM_B200_ERR_VOP; }
   if (!(d->rop <= 5 || d->rop == OP_UDEF)) { fprintf(stderr, "Unknown ROP Message\n"); return FUSEDMM_B200_ERR_ROP; }
   if (!(d->sop <= 1 || d->sop == OP_UDEF)) { fprintf(stderr, "Unknown SOP Message\n"); return FUSEDMM_B200_ERR_SOP; }
   if (!(d->vsc <= 2 || d->vsc == OP_UDEF)) { fprintf(stderr, "Unknown VSC Message\n"); return FUSEDMM_B200_ERR_VSC; }
   if (!(d->aop <= 3 || d->aop == OP_UDEF)) { fprintf(stderr, "Unknown AOP Message\n"); return FUSEDMM_B200_ERR_AOP; }
   if (d->vop == OP_UDEF || d->rop == OP_UDEF || d->vsc == OP_UDEF || d->aop == OP_UDEF) {
      fprintf(stderr, "fusedmm_b200: user-defined VOP/ROP/VSC/AOP functions are host code and cannot run on the GPU\n");
      return FUSEDMM_B200_ERR_UDEF;
   }
   if (d->vop == 0) d->vop = VOP_COPY_RHS;
   // the four messages the reference has optimised kernels for (fusedMM.c:523-594)
   d->pattern = PAT_GENERIC;
   if (d->aop == AOP_ADD && d->vop == VOP_COPY_RHS && d->rop == ROP_NOOP && d->sop == SOP_NOOP && d->vsc == VSC_NOOP) d->pattern = PAT_GCN;
   else if (d->aop == AOP_ADD && d->vop == VOP_COPY_RHS && d->rop == ROP_NOOP && d->sop == SOP_COPY && d->vsc == VSC_MUL) d->pattern = PAT_SPMM;
   else if (d->aop == AOP_ADD && d->vop == VOP_COPY_RHS && d->rop == ROP_DOT && d->sop == OP_UDEF && d->vsc == VSC_MUL) d->pattern = PAT_SIGMOID;
   else if (d->aop == AOP_ADD && d->vop == VOP_SUBR && d->rop == ROP_NORMR && d->sop == OP_UDEF && d->vsc == VSC_MUL) d->pattern = PAT_TDIST;
   return 0;
}

bool is_device_pointer(const void *p)
{
   if (!p) return false;
   cudaPointerAttributes a;
   if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
      cudaGetLastError();
      return false;
   }
   return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Default tiling for a row of `nvec` 16-byte vectors, from sweeps on B200 over the benchmark
// configurations (K = 64 .. 512, float and double).
void choose_tiling(long long nvec, bool is_double, int *G, int *NV, int *U)
{
   // *U also carries the register budget class of the instantiation in bits 8.. (fusedmm_inst.cuh)
   if (nvec <= 4) { *G = 4; *NV = 1; *U = 4; }
   else if (nvec <= 8) { *G = 8; *NV = 1; *U = 8; }
   else if (nvec <= 16) { *G = 8; *NV = 2; *U = 4 | (4 << 8); }
   else if (nvec <= 32) { *G = 16; *NV = 2; *U = 8; }
   else if (nvec <= 64) { *G = 32; *NV = 2; *U = is_double ? 8 : 4; }
   else if (nvec <= 128) { *G = 32; *NV = 4; *U = 2 | (3 << 8); }
   else if (nvec <= 256) { *G = 32; *NV = 8; *U = 1; }
   else if (nvec <= 512) { *G = 32; *NV = 16; *U = 1; }  // 2048 floats / 1024 doubles: X_u, Z_u and one gathered row = 192 registers
   else { *G = 0; *NV = 0; *U = 0; }
}
// The whole-row launch may use other gathers in flight / register budget than the chunk launch: its rows are short
// (at most `chunk` edges, on R-MAT graphs ten on average), so fewer gathers per slot are outstanding anyway and more
// resident warps pay more.  K = 128 floats on R-MAT scale 24: 43.7 ms per call with (16, 2, 4) in 80 registers for
// the whole rows against 45.4 with the chunk launch's (16, 2, 8) in 128.  false: use the chunk launch's tiling.
// With the whole rows sorted by length (option row_bins) two rows per warp pay for rows of 33..64 vectors as well:
// (16, 4, 2) in 80 registers, K = 128 doubles on R-MAT scale 24 75.8 ms against 80.5 with (32, 2, 4), K = 256 floats on
// scale 20 3.77 against 3.91 (without the sorting it loses: 89.8 against 85.9 and 4.70 against 4.29); K = 512 floats
// stays with one row per warp ((16, 8, 1): 24.4-25.0 ms against 24.4).
bool choose_rows_tiling(long long nvec, bool is_double, bool binned, int *G, int *NV, int *U)
{
   if (binned && nvec > 32 && nvec <= 64) { *G = 16; *NV = 4; *U = 2 | (3 << 8); return true; }
   if (!is_double && nvec > 16 && nvec <= 32) { *G = 16; *NV = 2; *U = 4 | (3 << 8); return true; }
   // K = 128 doubles, same graph: 85.9 ms with (32, 2, 4) in 80 registers for the whole rows against 90.6 with (32, 2, 8)
   if (is_double && nvec > 32 && nvec <= 64) { *G = 32; *NV = 2; *U = 4 | (3 << 8); return true; }
   return false;
}
// The flag-interpreting kernels need more registers than the specialised ones, so their best register budget and
// number of gathers in flight differ (B200, float): K = 512 SpMM message 43.8 ms without the 80-register budget of
// (32, 4, 2) against 52.0 with it; K = 256 FR message 7.24 ms with an 80-register budget on (32, 2, 4) against 8.95
// without; K = 128 sigmoid message 22.8 ms with 4 gathers in flight on (16, 2) against 26.3 with 8; the 64-register
// budget of (8, 2, 4) helps both kinds (K = 64: 3.48 ms against 4.46).
void tiling_for_generic(int G, int NV, int *U)
{
   if (G == 32 && NV == 4) *U &= 0xFF;
   else if (G == 32 && NV == 2 && *U == 4) *U = 4 | (3 << 8);
   else if (G == 16 && NV == 2 && *U == 8) *U = 4;
}
// Register budget of a kernel built at run time (and of the exact-K instantiations).  For three tilings the offline
// compiler settles on 80 registers (with a few spilled values) without being asked to, and the tilings were tuned with
// that; NVRTC gives the same source 96-106 registers, one resident block fewer per SM, and so does the offline compiler
// once the bounds predicates are gone.  Ask for the 80-register budget explicitly there.
int jit_budget(int G, int NV, int U, int MB)
{
   if (MB == 0 && ((G == 32 && NV == 2 && U == 4) || (G == 32 && NV == 1 && U == 8) || (G == 16 && NV == 1 && U == 8))) return 3;
   return MB;
}
// U of the default instantiation of a (G, NV) tiling
int default_u(int G, int NV)
{
   if (G == 4) return 4;
   return NV >= 8 ? 1 : 8 / NV;
}

struct HostArgs {
   int32_t imessage;
   long long m, n, k, nnz;
   const void *val, *indx, *pntrb, *pntre, *x, *y;
   void *z;
   long long ldx, ldy, ldz;
   double beta;
   int ptr_bits, idx_bits;
   int n_peers;
   void *const *z_peers;
   void *z_multicast;
   const fusedmm_b200_plan *plan;
};

// extent (one past the largest edge position) of indx/val when they have to be staged
template <typename PT>
long long max_entry(const PT *a, long long m)
{
   long long mx = 0;
   for (long long i = 0; i < m; i++) mx = std::max<long long>(mx, a[i]);
   return mx;
}

constexpr int PIPE_BLOCKS = 8;  // row blocks of the copy-back pipeline (one counter word and one event each)
template <typename PT>
int shard_rows(int64_t m, int32_t nshards, const PT *pntrb, const PT *pntre, int64_t *bounds, int64_t row_weight = 0);

template <typename T>
int run_typed(DeviceCtx &c, const HostArgs &a, const Decoded &d, const fusedmm_b200_sop &sopk,
              cudaStream_t user_stream)
{
   const bool async = user_stream != nullptr;
   cudaStream_t st = async ? user_stream : c.stream;
   const size_t es = sizeof(T), ps = a.ptr_bits / 8, is = a.idx_bits / 8;

   const bool need_x = vop_reads_x(d.vop) || rop_reads_x(d.rop);
   const bool need_y = vop_reads_y(d.vop);
   const bool need_val = d.rop == ROP_NOOP && d.vsc != VSC_NOOP;
   if ((need_x && !a.x) || (need_y && (!a.y || !a.indx)) || (need_val && !a.val) || !a.z || !a.pntrb || !a.pntre)
      return FUSEDMM_B200_ERR_ARG;
   if (a.ldz < a.k || (need_x && a.ldx < a.k) || (need_y && a.ldy < a.k)) return FUSEDMM_B200_ERR_ARG;

   // accumulate?  (beta semantics: see "beta_mode" in fusedmm_b200.h)
   const bool opt_pattern = d.pattern != PAT_GENERIC;
   const int accumulate = (t_opt.beta_mode == 0 && opt_pattern) ? (a.beta != 0.0) : 1;

   // ---- residency and staging ----------------------------------------------------------------------
   std::unique_ptr<NvtxRange> stage_range(new NvtxRange("fusedmm_b200: residency + staging"));
   const void *dv[7] = {a.val, a.indx, a.pntrb, a.pntre, a.x, a.y, a.z};
   bool on_dev[7];
   const bool used[7] = {need_val, need_y, true, true, need_x, need_y, true};
   for (int i = 0; i < 7; i++) on_dev[i] = used[i] ? is_device_pointer(dv[i]) : true;
   if (async) {
      for (int i = 0; i < 7; i++)
         if (!on_dev[i]) return FUSEDMM_B200_ERR_ARG;
   } else {
      // A synchronous call runs on the library's own stream.  Device arrays may still be the target of
      // work the caller enqueued on other streams (a fill, a copy): wait for the device first, so that
      // "synchronous" means what it means for the host function this replaces.
      bool any_dev = false;
      for (int i = 0; i < 7; i++) any_dev = any_dev || (used[i] && on_dev[i] && dv[i]);
      if (any_dev) CK(cudaDeviceSynchronize());
   }

   long long h2d = 0, d2h = 0;
   const bool pe_is_pb1 = (static_cast<const char *>(a.pntre) == static_cast<const char *>(a.pntrb) + ps);
   // A large Z that goes back to a host array is computed in blocks of rows (below).  With the usual (rowptr, rowptr+1)
   // row pointers on the host the edges of a block are one slice of indx / val, so those arrays follow block by block:
   // the slices of the later blocks come in while the earlier blocks compute and their rows of Z go out.
   const bool blocked_out = !a.plan && !async && !on_dev[6] && !on_dev[2] && !on_dev[3] &&
                            static_cast<size_t>(a.m) * a.k * es >= (static_cast<size_t>(32) << 20);
   const bool defer_edges = blocked_out && pe_is_pb1 && t_opt.blocked_inputs != 0;
   if (!on_dev[2] || !on_dev[3]) {
      if (!on_dev[2] && !on_dev[3] && pe_is_pb1) {
         CKI(ensure_buf(c.stage[2], (a.m + 1) * ps));
         CK(cudaMemcpyAsync(c.stage[2].ptr, a.pntrb, (a.m + 1) * ps, cudaMemcpyHostToDevice, st));
         dv[2] = c.stage[2].ptr;
         dv[3] = static_cast<char *>(c.stage[2].ptr) + ps;
         h2d += (a.m + 1) * ps;
      } else {
         for (int i = 2; i <= 3; i++)
            if (!on_dev[i]) {
               CKI(ensure_buf(c.stage[i], a.m * ps));
               CK(cudaMemcpyAsync(c.stage[i].ptr, i == 2 ? a.pntrb : a.pntre, a.m * ps, cudaMemcpyHostToDevice, st));
               dv[i] = c.stage[i].ptr;
               h2d += a.m * ps;
            }
      }
   }
   if ((need_y && !on_dev[1]) || (need_val && !on_dev[0])) {
      // number of edge slots the arrays span = largest pntre entry
      long long ext = 0;
      if (!on_dev[3]) {
         ext = a.ptr_bits == 64 ? max_entry(static_cast<const int64_t *>(a.pntre), a.m)
                                : max_entry(static_cast<const int32_t *>(a.pntre), a.m);
      } else {
         std::vector<char> tmp(a.m * ps);
         CK(cudaMemcpy(tmp.data(), a.pntre, a.m * ps, cudaMemcpyDeviceToHost));
         ext = a.ptr_bits == 64 ? max_entry(reinterpret_cast<const int64_t *>(tmp.data()), a.m)
                                : max_entry(reinterpret_cast<const int32_t *>(tmp.data()), a.m);
      }
      if (need_y && !on_dev[1]) {
         CKI(ensure_buf(c.stage[1], ext * is));
         if (!defer_edges) CK(cudaMemcpyAsync(c.stage[1].ptr, a.indx, ext * is, cudaMemcpyHostToDevice, st));
         dv[1] = c.stage[1].ptr;
         if (!defer_edges) h2d += ext * is;
      }
      if (need_val && !on_dev[0]) {
         CKI(ensure_buf(c.stage[0], ext * es));
         if (!defer_edges) CK(cudaMemcpyAsync(c.stage[0].ptr, a.val, ext * es, cudaMemcpyHostToDevice, st));
         dv[0] = c.stage[0].ptr;
         if (!defer_edges) h2d += ext * es;
      }
   }
   const long long xbytes = need_x && a.m > 0 ? ((a.m - 1) * a.ldx + a.k) * es : 0;
   const long long ybytes = need_y && a.n > 0 ? ((a.n - 1) * a.ldy + a.k) * es : 0;
   if (need_y && !on_dev[5]) {
      if (a.n <= 0) return FUSEDMM_B200_ERR_ARG;  // n bounds the copy of a host Y
      CKI(ensure_buf(c.stage[5], ybytes));
      CK(cudaMemcpyAsync(c.stage[5].ptr, a.y, ybytes, cudaMemcpyHostToDevice, st));
      dv[5] = c.stage[5].ptr;
      h2d += ybytes;
   }
   if (need_x && !on_dev[4]) {
      if (need_y && !on_dev[5] && a.x == a.y && a.ldx == a.ldy && xbytes <= ybytes) {
         dv[4] = dv[5];  // X and Y are the same host matrix (embedding case): one copy serves both
      } else {
         CKI(ensure_buf(c.stage[4], xbytes));
         CK(cudaMemcpyAsync(c.stage[4].ptr, a.x, xbytes, cudaMemcpyHostToDevice, st));
         dv[4] = c.stage[4].ptr;
         h2d += xbytes;
      }
   }
   long long zld = a.ldz;
   if (!on_dev[6]) {
      // staged Z is packed (ld = k) so that only the k used columns of each row travel
      zld = a.k;
      CKI(ensure_buf(c.stage[6], a.m * a.k * es));
      dv[6] = c.stage[6].ptr;
      if (accumulate) {
         if (a.ldz == a.k) CK(cudaMemcpyAsync(c.stage[6].ptr, a.z, a.m * a.k * es, cudaMemcpyHostToDevice, st));
         else CK(cudaMemcpy2DAsync(c.stage[6].ptr, a.k * es, a.z, a.ldz * es, a.k * es, a.m, cudaMemcpyHostToDevice, st));
         h2d += a.m * a.k * es;
      }
   }

   stage_range.reset();
   // ---- kernel parameters -----------------------------------------------------------------------------
   Params<T> p;
   memset(&p, 0, sizeof(p));
   p.val = static_cast<const T *>(dv[0]);
   p.indx = dv[1];
   p.pntrb = dv[2];
   p.pntre = dv[3];
   p.x = static_cast<const T *>(dv[4]);
   p.y = static_cast<const T *>(dv[5]);
   p.z = static_cast<T *>(const_cast<void *>(dv[6]));
   p.m = a.m; p.k = a.k; p.ldx = a.ldx; p.ldy = a.ldy; p.ldz = zld;
   p.ptr64 = a.ptr_bits == 64; p.idx64 = a.idx_bits == 64;
   p.vop = d.vop; p.rop = d.rop; p.sop = d.sop; p.vsc = d.vsc; p.aop = d.aop;
   p.sop_kind = sopk.kind;
   p.sp0 = static_cast<T>(sopk.p0); p.sp1 = static_cast<T>(sopk.p1); p.sp2 = static_cast<T>(sopk.p2);
   p.accumulate = accumulate;
   p.chunk = std::max<int64_t>(32, t_opt.hub_chunk);
   // Shorter pieces for small graphs (more work items, shorter critical path): measured on R-MAT graphs of
   // 2-260 M edges, 128 wins below about 16 M edges unless rows are long in bytes, 256 is within 1 % of the
   // best everywhere else.  nnz is only a hint here (the reference never reads it); a wrong value costs
   // speed, not correctness.
   if (a.nnz > 0 && a.nnz < (1ll << 24) && static_cast<size_t>(a.k) * es <= 1024) p.chunk = std::min<long long>(p.chunk, 128);
   // below about two million edges the call is a chain of latencies, and the longest whole row is one link of it:
   // R-MAT scale 14, K = 128, L2 flushed: 55 us per call with rows split at 64 edges, 59 at 128, 80 at 32
   if (a.nnz > 0 && a.nnz < (1ll << 21) && static_cast<size_t>(a.k) * es <= 1024) p.chunk = std::min<long long>(p.chunk, 64);
   if (a.plan) p.chunk = a.plan->chunk;  // the split-row list of a plan was made for this chunk size
   p.n_peers = 0;
   p.z_mc = nullptr;
   if (a.z_multicast) {
      if (!on_dev[6]) return FUSEDMM_B200_ERR_ARG;
      p.z_mc = static_cast<T *>(a.z_multicast);
   } else if (a.n_peers > 0) {
      // finished rows are also stored into the peers' Z buffers (same layout as z): only meaningful for
      // device-resident Z, and only the row scheduler's kernels carry the extra stores
      if (!on_dev[6] || a.n_peers > 8 || !a.z_peers) return FUSEDMM_B200_ERR_ARG;
      p.n_peers = a.n_peers;
      for (int i = 0; i < a.n_peers; i++) {
         if (!a.z_peers[i]) return FUSEDMM_B200_ERR_ARG;
         p.z_peer[i] = static_cast<T *>(a.z_peers[i]);
      }
   }
   p.skip_empty_remote = (p.z_mc || p.n_peers > 0) && t_opt.multi_skip_empty_rows;
   if (d.sop == OP_UDEF && sopk.kind == FUSEDMM_SOP_SIGMOID_TABLE_C) {
      DevBuf &tb = sizeof(T) == 4 ? c.table_f : c.table_d;
      if (!tb.ptr) {
         std::vector<T> host;
         build_sigmoid_table(host);
         CKI(ensure_buf(tb, host.size() * es));
         CK(cudaMemcpy(tb.ptr, host.data(), host.size() * es, cudaMemcpyHostToDevice));
      }
      p.sop_table = static_cast<const T *>(tb.ptr);
   }

   // ---- engine choice ---------------------------------------------------------------------------------
   auto aligned16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
   constexpr int W16 = VecOf<T>::W;  // elements per 16-byte vector
   bool vec_ok = (a.k % W16 == 0) && (zld % W16 == 0) && aligned16(p.z) &&
                 (!need_x || ((a.ldx % W16 == 0) && aligned16(p.x))) &&
                 (!need_y || ((a.ldy % W16 == 0) && aligned16(p.y)));
   for (int i = 0; i < p.n_peers; i++) vec_ok = vec_ok && aligned16(p.z_peer[i]);
   if (p.z_mc) vec_ok = vec_ok && aligned16(p.z_mc);
   // Rows that are not 16-byte granular (K, a leading dimension or a base address): the same engine with one-element
   // vectors (FLAG_ELEMENT) as long as a row fits its widest tiling (512 elements); beyond, the element-strided engine.
   const bool element_mode = !vec_ok && a.k <= 512 && t_opt.element_vectors && t_opt.engine != 2;
   if (element_mode) vec_ok = true;
   const int W = element_mode ? 1 : W16;  // elements per vector of the kernels this call launches
   int G = 0, NV = 0, U = 0;
   int Us = 0;  // gathers in flight and register budget of a kernel specialised for the message (U is the flag-interpreting kernel's)
   const int warps = static_cast<int>(std::min<int64_t>(std::max<int64_t>(t_opt.warps_per_cta, 1), WARPS_PER_CTA));
   if (vec_ok) {
      if (t_opt.force_tiling) {
         G = static_cast<int>((t_opt.force_tiling >> 8) & 0xFF);
         NV = static_cast<int>(t_opt.force_tiling & 0xFF);
         U = static_cast<int>((t_opt.force_tiling >> 16) & 0xFF);
         if (U == 0) U = default_u(G, NV);
         U |= static_cast<int>((t_opt.force_tiling >> 24) & 0xFF) << 8;  // register budget class (0 = default)
      } else {
         // one-element vectors: the table by elements, float's choices for both value types (one set of instantiations)
         choose_tiling(a.k / W, sizeof(T) == 8 && !element_mode, &G, &NV, &U);
         Us = U;
         if ((t_opt.force_generic || d.pattern == PAT_GENERIC) && !element_mode) tiling_for_generic(G, NV, &U);
      }
      if (Us == 0) Us = U;
      if (G == 0 || static_cast<long long>(G) * NV * W < a.k) vec_ok = false;
   }
   // Whole rows sorted by length inside windows (option row_bins: 0 never, 1 for graphs of 4 M edges and more, 2
   // always; a plan has sorted them when it was made), for launches in which several rows share a warp; never for a
   // call that could not name its rows in 32 bits.
   const long long est_edges = a.nnz > 0 ? a.nnz : a.m * 16;
   const bool bins_wanted = vec_ok && a.m < (1ll << 32) &&
                            (a.plan ? (a.plan->row_order != nullptr && t_opt.row_bins != 0)
                                    : (t_opt.row_bins == 2 || (t_opt.row_bins == 1 && est_edges >= (1ll << 22))));
   // the whole-row launch may use a tiling of its own (short rows are latency-bound, chunks throughput-bound)
   int Gr = G, NVr = NV, Ur = U, Urs = Us;  // Urs: U | budget of a specialised kernel for the whole rows
   if (vec_ok && !element_mode && !t_opt.force_tiling && !t_opt.force_tiling_rows) {
      int g2 = 0, nv2 = 0, u2 = 0;
      if (choose_rows_tiling(a.k / W, sizeof(T) == 8, bins_wanted, &g2, &nv2, &u2) && static_cast<long long>(g2) * nv2 * W >= a.k) {
         if (d.pattern != PAT_GENERIC && !t_opt.force_generic) { Gr = g2; NVr = nv2; Ur = u2; Urs = u2; }
         else if (g2 == G && nv2 == NV) Urs = u2;  // the flag-interpreting kernel keeps its own; one built for the message takes it
      }
   }
   if (vec_ok && t_opt.force_tiling_rows) {
      Gr = static_cast<int>((t_opt.force_tiling_rows >> 8) & 0xFF);
      NVr = static_cast<int>(t_opt.force_tiling_rows & 0xFF);
      Ur = static_cast<int>((t_opt.force_tiling_rows >> 16) & 0xFF);
      if (Ur == 0) Ur = default_u(Gr, NVr);
      Ur |= static_cast<int>((t_opt.force_tiling_rows >> 24) & 0xFF) << 8;
      Urs = Ur;
      if (Gr == 0 || 32 % Gr != 0 || static_cast<long long>(Gr) * NVr * W < a.k) return FUSEDMM_B200_ERR_ARG;
   }
   const int pattern = t_opt.force_generic ? PAT_GENERIC : d.pattern;
   // A message without a built-in specialised kernel gets one built at run time (fusedmm_jit.cu) when the policy of
   // option "jit" says it is worth it; otherwise, or when that fails, the flag-interpreting instantiation runs.
   const long long jit_weight = a.nnz > 0 && a.nnz < (1ll << 40) ? a.nnz * a.k : 0;
   int jit_policy = ((d.pattern == PAT_GENERIC && !t_opt.force_generic) || t_opt.force_generic == 2) ? static_cast<int>(t_opt.jit) : 0;
   // Flags of the CALL that pick a variant of the kernel (fusedmm_kernels.cuh): FLAG_ELEMENT for rows that are not
   // 16-byte granular; FLAG_EXACT_K, decided per launch in launch_main, when K fills the tiling exactly (compiled in
   // for the default tilings, built at run time for messages outside the four patterns); FLAG_OFFSET32 (32-bit row
   // offsets) only as an experiment behind option "jit_call_shape", always through a kernel built at run time.
   int jit_flags = element_mode ? FLAG_ELEMENT : 0;
   if (vec_ok && !element_mode && t_opt.jit_call_shape && t_opt.jit > 0 && !t_opt.force_generic && (jit_weight >= (1ll << 26) || t_opt.jit_call_shape == 2)) {
      const bool need_y_ = vop_reads_y(d.vop);
      if (need_y_ && a.idx_bits == 32 && static_cast<double>(a.ldy) * es < 4294967296.0)
         jit_flags |= FLAG_OFFSET32;
      jit_flags &= static_cast<int>(t_opt.jit_shape_mask);
      if (jit_flags & FLAG_OFFSET32) jit_policy = std::max<int>(jit_policy, static_cast<int>(t_opt.jit));
   }
   bool jit_used = false, bulk_used = false;
   auto launch_main = [&](const Params<T> &q, int g, int nv, int u_rt, int u_special, int w, long long grid, cudaStream_t s) -> bool {
      const bool ex = t_opt.exact_k && !element_mode && static_cast<long long>(g) * nv * W == a.k;  // per launch: the whole rows may have their own tiling
      const int fl = (jit_flags & ~FLAG_EXACT_K) | (ex ? FLAG_EXACT_K : 0);
      if (jit_policy > 0 && jit_launch_vec<T>(d.vop, d.rop, d.vsc, d.aop, g, nv, u_special & 0xFF,
                                              jit_budget(g, nv, u_special & 0xFF, u_special >> 8), fl, w, q, grid, s, jit_policy,
                                              jit_weight)) {
         jit_used = true;
         return true;
      }
      if (t_opt.offset32 && need_y && !element_mode && a.idx_bits == 32 && static_cast<double>(a.ldy) * es < 4294967296.0 &&
          q.mode == MODE_ROWS) {
         // 32-bit column ids: the variant with the one-instruction row address, for the tiling that has one (fusedmm_inst.cuh)
         const int u_budget = (u_rt & 0xFF) | (jit_budget(g, nv, u_rt & 0xFF, (u_rt >> 8) & 0xFF) << 8);
         if (ex && launch_vec<T>(pattern, g, nv, u_budget | (5 << 16), w, q, grid, s)) return true;
         if (ex && launch_vec<T>(pattern, g, nv, u_rt | (5 << 16), w, q, grid, s)) return true;
         if (!ex && launch_vec<T>(pattern, g, nv, u_rt | (4 << 16), w, q, grid, s)) return true;
      }
      if (fl & FLAG_EXACT_K) {
         // without the predicates the offline compiler no longer settles on 80 registers for (32, 2, 4) by itself (93):
         // ask for the budget the tiling was tuned with
         const int u_budget = (u_rt & 0xFF) | (jit_budget(g, nv, u_rt & 0xFF, (u_rt >> 8) & 0xFF) << 8);
         if (launch_vec<T>(pattern, g, nv, u_budget | (1 << 16), w, q, grid, s)) return true;
         if (launch_vec<T>(pattern, g, nv, u_rt | (1 << 16), w, q, grid, s)) return true;
      }
      if (launch_vec<T>(pattern, g, nv, u_rt | (element_mode ? (2 << 16) : 0), w, q, grid, s)) return true;
      // a tiling (option force_tiling / force_tiling_rows) that is not among the instantiations compiled into the
      // library: build it at run time
      if (t_opt.jit > 0 && g > 0 && 32 % g == 0 && nv > 0 && (u_rt & 0xFF) > 0 &&
          jit_launch_vec<T>(d.vop, d.rop, d.vsc, d.aop, g, nv, u_rt & 0xFF, u_rt >> 8, element_mode ? FLAG_ELEMENT : 0, w, q, grid, s, 2,
                            jit_weight)) {
         jit_used = true;
         return true;
      }
      return false;
   };

   int launches = 0;
   bool z_returned = false;  // the blocked path below has already copied Z back to the host
   float ms = 0.f, ms_k[4] = {0.f, 0.f, 0.f, 0.f}, ms_main = 0.f;
   long long nh = 0, nchunks = 0;
   // The edge-stream scheduler needs row r+1 to start where row r ends, which the usual
   // (rowptr, rowptr+1) way of passing pntrb/pntre guarantees; anything else takes the row scheduler.
   const bool contiguous_rows = static_cast<const char *>(dv[3]) == static_cast<const char *>(dv[2]) + ps;
   const bool use_stream = vec_ok && contiguous_rows && t_opt.engine == 2 && p.n_peers == 0 && !p.z_mc && !a.plan && NV <= 8;
   p.counter = static_cast<unsigned long long *>(c.counter.ptr);
   p.error = static_cast<unsigned long long *>(c.counter.ptr) + 12;  // word 12 of the counter block: "a bounded wait ran out"

   if (use_stream) {
      // ---- edge-stream scheduler: partition, main kernel, fix-up ------------------------------------
      p.quantum = (t_opt.edge_quantum + 31) / 32 * 32;
      int depth = std::min(G, 8);  // at least one segment; a power of two <= 32
      while (depth * 2 <= std::min<int64_t>(t_opt.stream_depth, 32)) depth *= 2;
      p.depth = depth;
      if (c.part_cap == 0 || c.heads.bytes == 0) {
         long long want = 1 << 16;
         if (a.nnz > 0 && a.nnz < (1ll << 38)) {  // nnz is only a sizing hint (the reference never reads it)
            size_t free_b = 0, total_b = 0;
            CK(cudaMemGetInfo(&free_b, &total_b));
            const long long hint = a.nnz / p.quantum + 2;
            if (static_cast<double>(hint) * a.k * es < 0.25 * static_cast<double>(free_b)) want = std::max(want, hint);
         }
         c.part_cap = std::max(c.part_cap, want);
      }
      for (int attempt = 0; attempt < 3; attempt++) {
         CKI(ensure_buf(c.part, (c.part_cap + 1) * sizeof(long long)));
         CKI(ensure_buf(c.heads, static_cast<size_t>(c.part_cap) * a.k * es));
         p.part = static_cast<long long *>(c.part.ptr);
         p.heads = static_cast<T *>(c.heads.ptr);
         p.part_cap = std::min<long long>(c.part_cap, static_cast<long long>(c.heads.bytes / (static_cast<size_t>(a.k) * es)));
         if (!async) CK(cudaEventRecord(c.ev0, st));
         stream_partition_kernel<T><<<c.sm_count * 8, 256, 0, st>>>(p);
         if (!async) CK(cudaEventRecord(c.evk[0], st));
         int swarps = warps;  // the ring of every warp must fit into the shared memory of one SM
         while (swarps > 1 && static_cast<size_t>(swarps) * p.depth * NV * 512 > (static_cast<size_t>(96) << 10)) swarps /= 2;
         if (!launch_stream<T>(pattern, G, NV, swarps, p, c.sm_count, st)) return FUSEDMM_B200_ERR_ARG;
         if (!async) CK(cudaEventRecord(c.evk[1], st));
         stream_fixup_kernel<T><<<c.sm_count * 4, WARPS_PER_CTA * 32, 0, st>>>(p);
         launches += 3;
         CK(cudaGetLastError());
         if (async) {
            c.async_pending = true;
            c.async_engine = 2;
            c.async_k = a.k;
            c.async_elt = es;
            break;
         }
         CK(cudaEventRecord(c.ev1, st));
         unsigned long long nq = 0;
         CK(cudaMemcpyAsync(&nq, static_cast<unsigned long long *>(c.counter.ptr) + 1, sizeof(nq), cudaMemcpyDeviceToHost, st));
         CK(cudaStreamSynchronize(st));
         float t = 0.f;
         CK(cudaEventElapsedTime(&t, c.ev0, c.ev1)); ms += t;
         CK(cudaEventElapsedTime(&t, c.ev0, c.evk[0])); ms_k[0] += t;
         CK(cudaEventElapsedTime(&t, c.evk[0], c.evk[1])); ms_k[1] += t;
         CK(cudaEventElapsedTime(&t, c.evk[1], c.ev1)); ms_k[3] += t;
         CK(cudaEventElapsedTime(&t, c.evk[0], c.ev1)); ms_main += t;
         nchunks = static_cast<long long>(nq);
         if (nchunks <= p.part_cap) break;
         if (attempt == 2) return FUSEDMM_B200_ERR_LIMIT;
         c.part_cap = nchunks + nchunks / 16 + 64;  // nothing but zero rows was written; enlarge and rerun
      }
   } else {
   // ---- row scheduler: whole rows, chunks of long rows, fix-up ----------------------------------------
   if (c.hub_cap == 0) {
      c.hub_cap = std::max<int64_t>(16, t_opt.hub_cap_initial);
      CKI(ensure_buf(c.hub_row, c.hub_cap * sizeof(long long)));
      CKI(ensure_buf(c.hub_base, c.hub_cap * sizeof(long long)));
   }
   if (c.partials.bytes == 0) CKI(ensure_buf(c.partials, static_cast<size_t>(64) << 20));
   if (!a.plan && a.nnz > 0 && a.nnz < (1ll << 38)) {
      // With a truthful nnz the scratch can be sized before anything runs (a row is split only if it has
      // more than `chunk` edges), so that a call enqueued on a caller's stream never finds it too small.
      // nnz stays a hint: if it understates the graph the overflow path below still catches it.
      const long long bound_hubs = a.nnz / p.chunk + 1, bound_chunks = a.nnz / p.chunk + bound_hubs;
      const size_t want = static_cast<size_t>(bound_chunks) * a.k * es;
      if (bound_hubs > c.hub_cap || want > c.partials.bytes) {
         size_t free_b = 0, total_b = 0;
         CK(cudaMemGetInfo(&free_b, &total_b));
         if (static_cast<double>(want) < 0.25 * static_cast<double>(free_b)) {
            if (bound_hubs > c.hub_cap) {
               c.hub_cap = bound_hubs;
               CKI(ensure_buf(c.hub_row, c.hub_cap * sizeof(long long)));
               CKI(ensure_buf(c.hub_base, c.hub_cap * sizeof(long long)));
            }
            CKI(ensure_buf(c.partials, want));
         }
      }
   }
   const long long rows_per_warp = vec_ok ? 32 / Gr : 1;  // short rows: one per group of lanes
   const long long hub_grid = static_cast<long long>(c.sm_count) * t_opt.chunk_ctas_per_sm;
   // Chunks visited in the order of their first column id (option chunk_order: 0 never, 1 when the graph is large
   // enough for the three launches of the sort to pay, 2 always).  Measured on R-MAT graphs: 16 M edges with K = 512
   // floats 28.4 -> 24.3 ms, 520 M edges with K = 128 41.8 -> 40.0 ms, 31 M edges with K = 256 3.96 -> 3.91 ms,
   // 0.4 M edges 59 -> 87 us.
   bool use_bins = !a.plan && bins_wanted && Gr < 32;
   bool use_order = !a.plan && need_y && (t_opt.chunk_order == 2 || (t_opt.chunk_order == 1 && est_edges >= (1ll << 24)));

   // One pass of the row scheduler over the rows that `q` describes: scan, then the chunks of split rows
   // (and their fix-up) on the side stream beside the whole rows on `st`, forked after the scan and joined
   // before `st` continues.
   auto enqueue_pass = [&](Params<T> &q, bool with_rows, bool timing) -> int {
      NvtxRange pass_range("fusedmm_b200: row scheduler pass (rows || scan -> chunks -> fix-up)");
      const long long qgrid = (q.m + warps * rows_per_warp - 1) / (warps * rows_per_warp);
      // The whole rows need nothing from the scan, so they start at once on `st`; the scan, the chunks of the split
      // rows and the fix-up form a chain on the side stream, each launched so that it can become resident while its
      // predecessor drains (programmatic dependent launch).
      if (timing) CK(cudaEventRecord(c.evk[0], st));
      CK(cudaEventRecord(c.ev_fork, st));
      cudaStream_t side = !t_opt.side_stream ? st : (t_opt.side_priority ? c.side_hi : c.side);
      CK(cudaStreamWaitEvent(side, c.ev_fork, 0));
      const bool pdl = t_opt.pdl != 0;
      if (!a.plan) {  // a plan carries the result of this scan
         CK(cudaMemsetAsync(q.counter, 0, sizeof(unsigned long long), side));
         scan_hub_rows<<<static_cast<unsigned int>((q.m + 255) / 256), 256, 0, side>>>(
            q.pntrb, q.pntre, q.ptr64, q.m, q.chunk, q.counter, q.hub_row, q.hub_base, q.hub_cap);
         launches++;
      }
      if (!a.plan) q.order = nullptr;
      if (use_order && c.order.bytes >= static_cast<size_t>(q.chunk_cap) * sizeof(long long)) {
         CK(enqueue_chunk_order(q.pntrb, q.pntre, q.ptr64, q.indx, q.idx64, a.n > 0 ? a.n : a.m, q.chunk, q.counter, q.hub_row,
                                q.hub_base, q.hub_cap, q.chunk_cap, static_cast<unsigned int *>(c.order_cnt.ptr),
                                static_cast<long long *>(c.order.ptr), c.sm_count, side));
         q.order = static_cast<const long long *>(c.order.ptr);
         launches += 3;
      }
      // events between the kernels of the chain (option timing_detail) would undo the pairing of the launches
      const bool detail = timing && t_opt.timing_detail;
      if (detail) CK(cudaEventRecord(c.evk[2], side));
      q.mode = MODE_HUB_CHUNKS;
      q.pdl = pdl && !a.plan && !detail;
      bool chunks_launched = false;
      if (vec_ok && !element_mode && t_opt.bulk_chunks && need_y && pattern != PAT_GENERIC) {
         // option bulk_chunks: neighbour rows staged through shared memory by bulk copies (fusedmm_bulk.cuh)
         const int bw = static_cast<int>(std::min<int64_t>(std::max<int64_t>(t_opt.bulk_warps, 1), WARPS_PER_CTA));
         chunks_launched = launch_bulk<T>(pattern, G, NV, static_cast<int>(t_opt.bulk_chunks), bw, q, c.sm_count,
                                          static_cast<int>(t_opt.bulk_ctas_per_sm), side);
         bulk_used = bulk_used || chunks_launched;
      }
      if (!chunks_launched) {
         if (vec_ok) { if (!launch_main(q, G, NV, U, Us, WARPS_PER_CTA, hub_grid, side)) return FUSEDMM_B200_ERR_ARG; }
         else launch_any<T>(q, WARPS_PER_CTA, hub_grid, side);
      }
      if (detail) CK(cudaEventRecord(c.evk[3], side));
      q.pdl = pdl && !detail;
      launch_fixup<T>(q, static_cast<long long>(c.sm_count) * 4, side);
      q.pdl = 0;
      if (detail) CK(cudaEventRecord(c.ev_side_end, side));
      CK(cudaEventRecord(c.ev_join, side));
      launches += 2;
      if (with_rows) {  // whole rows only once: a rerun after a scratch overflow redoes split rows only
         q.mode = MODE_ROWS;
         if (!a.plan) q.row_order = nullptr;
         if (use_bins && q.m > 0) {
            bin_rows_kernel<<<static_cast<unsigned int>((q.m + ROW_BIN_TILE - 1) / ROW_BIN_TILE), 256, 0, st>>>(
               q.pntrb, q.pntre, q.ptr64, q.m, q.chunk, static_cast<unsigned int *>(c.row_order.ptr));
            q.row_order = static_cast<const unsigned int *>(c.row_order.ptr);
            launches++;
         }
         if (vec_ok) { if (!launch_main(q, Gr, NVr, Ur, Urs, warps, qgrid, st)) return FUSEDMM_B200_ERR_ARG; }
         else launch_any<T>(q, warps, qgrid, st);
         launches++;
      }
      if (detail) CK(cudaEventRecord(c.evk[1], st));
      CK(cudaStreamWaitEvent(st, c.ev_join, 0));
      CK(cudaGetLastError());
      return 0;
   };
   auto bind_scratch = [&](Params<T> &q) {
      q.hub_row = a.plan ? a.plan->hub_row : static_cast<long long *>(c.hub_row.ptr);
      q.hub_base = a.plan ? a.plan->hub_base : static_cast<long long *>(c.hub_base.ptr);
      q.hub_cap = a.plan ? std::max<long long>(a.plan->nh, 1) : c.hub_cap;
      if (a.plan) q.counter = a.plan->counter;
      if (a.plan) q.order = (need_y && t_opt.chunk_order != 0) ? a.plan->order : nullptr;
      q.partials = static_cast<T *>(c.partials.ptr);
      q.chunk_cap = static_cast<long long>(c.partials.bytes / (static_cast<size_t>(a.k) * es));
      if (use_bins && ensure_buf(c.row_order, static_cast<size_t>(a.m) * sizeof(unsigned int))) use_bins = false;
      if (a.plan) q.row_order = (bins_wanted && Gr < 32) ? a.plan->row_order : nullptr;
      if (use_order) {
         if (ensure_buf(c.order, static_cast<size_t>(q.chunk_cap) * sizeof(long long))) use_order = false;
         if (ensure_buf(c.order_cnt, 3 * ORDER_BUCKETS * sizeof(unsigned int))) use_order = false;
      }
   };

   // ---- Z goes back to a host array: copy it block of rows by block of rows while later blocks compute ----
   if (a.plan) CKI(ensure_buf(c.partials, static_cast<size_t>(std::max<long long>(a.plan->nchunks, 1)) * a.k * es));
   if (blocked_out) {
      int64_t bounds[PIPE_BLOCKS + 1];
      CKI(a.ptr_bits == 64 ? shard_rows(a.m, PIPE_BLOCKS, static_cast<const int64_t *>(a.pntrb), static_cast<const int64_t *>(a.pntre), bounds)
                           : shard_rows(a.m, PIPE_BLOCKS, static_cast<const int32_t *>(a.pntrb), static_cast<const int32_t *>(a.pntre), bounds));
      if (defer_edges) {
         // the slices follow the dense inputs on the link, in block order; block b's kernels wait for slice b only
         auto row_start = [&](int64_t r) -> long long {  // rowptr has m + 1 entries here (pntre == pntrb + 1)
            return a.ptr_bits == 64 ? static_cast<long long>(static_cast<const int64_t *>(a.pntrb)[r])
                                    : static_cast<long long>(static_cast<const int32_t *>(a.pntrb)[r]);
         };
         // (the first slice does not wait for them: it shares the link with the dense inputs, so the first block can
         // start the moment those have arrived)
         CK(cudaEventRecord(c.ev_inputs, st));
         const bool in_idx = need_y && !on_dev[1], in_val = need_val && !on_dev[0];
         const long long cap_e = std::min<long long>(in_idx ? static_cast<long long>(c.stage[1].bytes / is) : (1ll << 62),
                                                     in_val ? static_cast<long long>(c.stage[0].bytes / es) : (1ll << 62));
         for (int b = 0; b < PIPE_BLOCKS; b++) {
            if (b == 1) CK(cudaStreamWaitEvent(c.copy_in, c.ev_inputs, 0));
            long long e0 = row_start(bounds[b]), e1 = row_start(bounds[b + 1]);
            e0 = std::max<long long>(0, std::min(e0, cap_e));
            e1 = std::max<long long>(e0, std::min(e1, cap_e));
            if (e1 > e0 && in_idx) {
               CK(cudaMemcpyAsync(static_cast<char *>(c.stage[1].ptr) + e0 * is, static_cast<const char *>(a.indx) + e0 * is, (e1 - e0) * is,
                                  cudaMemcpyHostToDevice, c.copy_in));
               h2d += (e1 - e0) * is;
            }
            if (e1 > e0 && in_val) {
               CK(cudaMemcpyAsync(static_cast<char *>(c.stage[0].ptr) + e0 * es, static_cast<const char *>(a.val) + e0 * es, (e1 - e0) * es,
                                  cudaMemcpyHostToDevice, c.copy_in));
               h2d += (e1 - e0) * es;
            }
            CK(cudaEventRecord(c.ev_in[b], c.copy_in));
         }
      }
      // One block: its rows through the row scheduler (whole rows only on the first pass), then its part of Z back
      // to the host on the copy stream while the next block computes.
      auto run_block = [&](int b, bool with_rows) -> int {
         const long long r0 = bounds[b], r1 = bounds[b + 1];
         if (r1 <= r0) return 0;
         Params<T> q = p;
         q.m = r1 - r0;
         q.pntrb = static_cast<const char *>(p.pntrb) + r0 * ps;
         q.pntre = static_cast<const char *>(p.pntre) + r0 * ps;
         if (q.x) q.x = p.x + r0 * p.ldx;
         q.z = p.z + r0 * p.ldz;
         q.counter = p.counter + 2 + b;  // words 0 and 1 belong to the unblocked passes
         if (defer_edges && with_rows) CK(cudaStreamWaitEvent(st, c.ev_in[b], 0));  // first pass: this block's slice has arrived
         CKI(enqueue_pass(q, with_rows, false));
         CK(cudaEventRecord(c.ev_block[b], st));
         CK(cudaStreamWaitEvent(c.copy, c.ev_block[b], 0));
         const char *src = static_cast<const char *>(c.stage[6].ptr) + static_cast<size_t>(r0) * a.k * es;
         char *dst = static_cast<char *>(a.z) + static_cast<size_t>(r0) * a.ldz * es;
         if (a.ldz == a.k) CK(cudaMemcpyAsync(dst, src, static_cast<size_t>(r1 - r0) * a.k * es, cudaMemcpyDeviceToHost, c.copy));
         else CK(cudaMemcpy2DAsync(dst, a.ldz * es, src, a.k * es, a.k * es, r1 - r0, cudaMemcpyDeviceToHost, c.copy));
         return 0;
      };
      bool redo[PIPE_BLOCKS];
      for (int b = 0; b < PIPE_BLOCKS; b++) redo[b] = true;
      for (int attempt = 0; attempt < 3; attempt++) {
         bind_scratch(p);
         for (int b = 0; b < PIPE_BLOCKS; b++)
            if (redo[b]) CKI(run_block(b, attempt == 0));
         unsigned long long words[PIPE_BLOCKS] = {};
         CK(cudaMemcpyAsync(words, p.counter + 2, sizeof(words), cudaMemcpyDeviceToHost, st));
         CK(cudaStreamSynchronize(st));
         CK(cudaStreamSynchronize(c.copy));
         // A block whose split rows did not fit has run its whole rows (once) and none of its split rows: only
         // those blocks are redone, split rows only, so that nothing is accumulated into Z twice; the blocks that
         // fitted are complete and already with the caller.
         bool fits = true;
         long long need_h = 0, need_c = 0;
         nh = nchunks = 0;
         for (int b = 0; b < PIPE_BLOCKS; b++) {
            if (bounds[b + 1] <= bounds[b]) { redo[b] = false; continue; }
            const long long bh = static_cast<long long>(words[b] >> HUB_SHIFT), bc = static_cast<long long>(words[b] & HUB_CHUNK_MASK);
            redo[b] = redo[b] && (bh > p.hub_cap || bc > p.chunk_cap);
            fits = fits && !redo[b];
            need_h = std::max(need_h, bh);
            need_c = std::max(need_c, bc);
            nh += bh;
            nchunks += bc;
         }
         if (fits) break;
         if (attempt == 2) return FUSEDMM_B200_ERR_LIMIT;
         if (need_h > c.hub_cap) {
            c.hub_cap = need_h + need_h / 4 + 1024;
            CKI(ensure_buf(c.hub_row, c.hub_cap * sizeof(long long)));
            CKI(ensure_buf(c.hub_base, c.hub_cap * sizeof(long long)));
         }
         if (need_c > p.chunk_cap) CKI(ensure_buf(c.partials, static_cast<size_t>(need_c + need_c / 8 + 64) * a.k * es));
      }
      z_returned = true;
      d2h += a.m * a.k * es;
   }

   for (int attempt = 0; attempt < 3 && !z_returned; attempt++) {
      bind_scratch(p);
      if (!async) CK(cudaEventRecord(c.ev0, st));
      CKI(enqueue_pass(p, attempt == 0, !async));
      if (async) {
         if (!a.plan) {  // the scratch of a plan call is sized exactly: nothing to report later
            c.async_pending = true;
            c.async_engine = 1;
            c.async_k = a.k;
            c.async_elt = es;
         }
         break;
      }
      CK(cudaEventRecord(c.ev1, st));
      unsigned long long packed = 0;
      CK(cudaMemcpyAsync(&packed, p.counter, sizeof(packed), cudaMemcpyDeviceToHost, st));
      CK(cudaStreamSynchronize(st));
      float t = 0.f;
      CK(cudaEventElapsedTime(&t, c.ev0, c.ev1));
      ms += t;
      if (t_opt.timing_detail) {
         CK(cudaEventElapsedTime(&t, c.evk[0], c.evk[2])); ms_k[0] += t;   // start of the pass -> scan done
         CK(cudaEventElapsedTime(&t, c.evk[0], c.evk[1])); ms_k[1] += t;   // whole rows, beside the chain
         CK(cudaEventElapsedTime(&t, c.evk[2], c.evk[3])); ms_k[2] += t;
         CK(cudaEventElapsedTime(&t, c.evk[3], c.ev_side_end)); ms_k[3] += t;
      }
      CK(cudaEventElapsedTime(&t, c.evk[0], c.ev1)); ms_main += t;
      nh = static_cast<long long>(packed >> HUB_SHIFT);
      nchunks = static_cast<long long>(packed & HUB_CHUNK_MASK);
      if (bulk_used) {  // a bounded wait of the bulk-copy kernel ran out: its result cannot be trusted
         unsigned long long err = 0;
         CK(cudaMemcpy(&err, p.error, sizeof(err), cudaMemcpyDeviceToHost));
         if (err) {
            CK(cudaMemset(p.error, 0, sizeof(err)));
            fprintf(stderr, "fusedmm_b200: a bulk copy did not complete within its wait limit\n");
            return FUSEDMM_B200_ERR_CUDA;
         }
      }
      if (nh <= p.hub_cap && nchunks <= p.chunk_cap) break;
      if (attempt == 2) return FUSEDMM_B200_ERR_LIMIT;
      // scratch was too small: the chunk and fix-up passes did nothing.  Enlarge and redo them.
      if (nh > c.hub_cap) {
         c.hub_cap = nh + nh / 4 + 1024;
         CKI(ensure_buf(c.hub_row, c.hub_cap * sizeof(long long)));
         CKI(ensure_buf(c.hub_base, c.hub_cap * sizeof(long long)));
      }
      if (nchunks > p.chunk_cap) CKI(ensure_buf(c.partials, static_cast<size_t>(nchunks + nchunks / 8 + 64) * a.k * es));
   }
   }

   if (!on_dev[6] && !z_returned) {
      NvtxRange copy_range("fusedmm_b200: Z back to the host");
      if (a.ldz == a.k) CK(cudaMemcpyAsync(a.z, c.stage[6].ptr, a.m * a.k * es, cudaMemcpyDeviceToHost, st));
      else CK(cudaMemcpy2DAsync(a.z, a.ldz * es, c.stage[6].ptr, a.k * es, a.k * es, a.m, cudaMemcpyDeviceToHost, st));
      CK(cudaStreamSynchronize(st));
      d2h += a.m * a.k * es;
   }
   t_info.kernel_launches = launches;
   t_info.pattern = pattern;
   t_info.lanes_per_edge = vec_ok ? G : 0;
   t_info.vectors_per_lane = vec_ok ? NV : 0;
   t_info.h2d_bytes = h2d;
   t_info.d2h_bytes = d2h;
   t_info.engine = use_stream ? 2 : 1;
   t_info.hub_rows = nh;
   t_info.hub_chunks = nchunks;
   t_info.device_ms = ms;
   t_info.ms_scan = ms_k[0]; t_info.ms_rows = ms_k[1]; t_info.ms_chunks = ms_k[2]; t_info.ms_fixup = ms_k[3];
   t_info.ms_main = ms_main;
   t_info.sop_kind = d.sop == OP_UDEF ? sopk.kind : -1;
   t_info.jit_kernel = jit_used ? 1 : 0;
   static const bool trace = getenv("FUSEDMM_B200_TRACE") != nullptr;
   if (trace)
      fprintf(stderr, "fusedmm_b200: msg=%#x %s m=%lld k=%lld engine=%d tiling=%dx%d launches=%d split_rows=%lld chunks=%lld "
                      "h2d=%lld d2h=%lld B device=%.3f ms (scan %.3f, rows %.3f, chunks %.3f, fix-up %.3f)%s\n",
              a.imessage, sizeof(T) == 4 ? "f32" : "f64", a.m, a.k, use_stream ? 2 : 1, vec_ok ? G : 0, vec_ok ? NV : 0, launches,
              nh, nchunks, h2d, d2h, ms, ms_k[0], ms_k[1], ms_k[2], ms_k[3], async ? " [enqueued]" : "");
   return 0;
}

// hook_kind: 0 none, 1 float hook, 2 double hook
int run_call(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage, int64_t m, int64_t n,
             int64_t k, int64_t nnz, const void *val, const void *indx, const void *pntrb, const void *pntre,
             const void *x, int64_t ldx, const void *y, int64_t ldy, double beta, void *z, int64_t ldz,
             const fusedmm_b200_sop *sop, void *hook, void *stream, int n_peers = 0, void *const *z_peers = nullptr,
             void *z_multicast = nullptr, const fusedmm_b200_plan *plan = nullptr)
{
   NvtxRange call_range("fusedmm_b200: fusedMM_csr");
   memset(&t_info, 0, sizeof(t_info));
   if ((dtype != 0 && dtype != 1) || (ptr_bits != 32 && ptr_bits != 64) || (idx_bits != 32 && idx_bits != 64))
      return FUSEDMM_B200_ERR_ARG;
   fusedmm_b200_sop sopk;
   {
      std::lock_guard<std::mutex> lock(g_mu);
      t_opt = g_opt;
      sopk = g_sop;
   }
   Decoded d;
   int st = decode_message(imessage, t_opt, &d);
   if (st) return st;
   if (d.sop == OP_UDEF) {
      if (sop) {
         if (sop->kind < 0 || sop->kind >= FUSEDMM_SOP_KIND_COUNT) return FUSEDMM_B200_ERR_UDEF;
         sopk = *sop;
      } else if (hook) {
         if (t_opt.strict_udef) {
            fprintf(stderr, "fusedmm_b200: option strict_udef is set: SOP_UDEF needs an explicit scalar function "
                            "(fusedmm_b200_set_sop or the sop argument), a host SOP_UDEF_FUNC is not examined\n");
            return FUSEDMM_B200_ERR_UDEF;
         }
         const bool ok = dtype == 0 ? identify_udef<float>(reinterpret_cast<int (*)(float, float *)>(hook), &sopk)
                                    : identify_udef<double>(reinterpret_cast<int (*)(double, double *)>(hook), &sopk);
         if (!ok) {
            fprintf(stderr, "fusedmm_b200: SOP_UDEF_FUNC is not one of the scalar functions the device implements "
                            "(see FUSEDMM_SOP_* in fusedmm_b200.h)\n");
            return FUSEDMM_B200_ERR_UDEF;
         }
         static std::atomic<bool> told{false};  // once per process: which device function stands in for the caller's host function
         if (getenv("FUSEDMM_B200_TRACE") && !told.exchange(true))
            fprintf(stderr, "fusedmm_b200: SOP_UDEF_FUNC matches built-in scalar function %d at the sample points "
                            "(FUSEDMM_SOP_* in fusedmm_b200.h); the device evaluates that function\n", sopk.kind);
      }
   }
   if (m < 0 || k < 0) return FUSEDMM_B200_ERR_ARG;
   if (d.aop == AOP_NOOP || m == 0 || k == 0) return 0;  // nothing is written to Z (fusedMM.c:268-273)
   DeviceCtx *c = nullptr;
   std::unique_lock<std::mutex> device_lock;
   CKI(enter_device(&c, &device_lock));
   HostArgs a = {imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, y, z, ldx, ldy, ldz, beta, ptr_bits, idx_bits, n_peers, z_peers, z_multicast, plan};
   return dtype == 0 ? run_typed<float>(*c, a, d, sopk, static_cast<cudaStream_t>(stream))
                     : run_typed<double>(*c, a, d, sopk, static_cast<cudaStream_t>(stream));
}

// =====================================================================================================
// The entry point that allocates nothing (fusedmm_b200_csr_static_scratch).
//
// Its split-row scratch (the hub list, the per-chunk partial sums, the packed counter, the sigmoid table)
// is this file-scope device array instead of buffers obtained from cudaMalloc.  Every GPU on which the
// library runs holds its own copy of the array from the moment the library is loaded until the process
// exits.  In host code the name below is only a stand-in for the symbol, NOT a device address: the address
// comes from cudaGetSymbolAddress, once per device, with that device current (static_scratch_base), and only
// that address is ever handed to a kernel.
// =====================================================================================================
#define FUSEDMM_B200_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[FUSEDMM_B200_STATIC_SCRATCH_BYTES];

constexpr int STATIC_MAX_DEVICES = 64;
constexpr long long STATIC_HUB_CAP = 32768;                    // split rows the hub list has room for
constexpr size_t STATIC_OFF_TABLE_F = 256;                     // after the packed counter: the float sigmoid table,
constexpr size_t STATIC_OFF_TABLE_D = STATIC_OFF_TABLE_F + SM_TABLE_SIZE * sizeof(float);  // then the double one
constexpr size_t STATIC_OFF_HUB_ROW = STATIC_OFF_TABLE_D + SM_TABLE_SIZE * sizeof(double);
constexpr size_t STATIC_OFF_HUB_BASE = STATIC_OFF_HUB_ROW + STATIC_HUB_CAP * sizeof(long long);
constexpr size_t STATIC_OFF_PARTIALS = STATIC_OFF_HUB_BASE + STATIC_HUB_CAP * sizeof(long long);
static_assert(STATIC_MAX_DEVICES == MAX_DEVICES, "one slot per device context");
static_assert(STATIC_OFF_PARTIALS % 256 == 0, "the partial sums must start on a 256-byte boundary");

struct StaticScratchSlot {
   unsigned char *base = nullptr;  // device address of g_static_scratch on this device
   int sm_count = 0;
   // caps of the latest call that was enqueued on a caller's stream, for fusedmm_b200_stream_status
   bool async_pending = false;
   long long async_hub_cap = 0, async_chunk_cap = 0;
};
StaticScratchSlot g_static_slot[STATIC_MAX_DEVICES];

template <typename T>
const T *static_host_sigmoid_table()
{
   static T table[SM_TABLE_SIZE];
   static bool ready = false;
   if (!ready) {
      for (int i = 0; i < SM_TABLE_SIZE; i++) {
         T x = static_cast<T>(2.0 * 5.0 * i / SM_TABLE_SIZE - 5.0);
         table[i] = static_cast<T>(1.0 / (1 + std::exp(-static_cast<double>(x))));
      }
      ready = true;
   }
   return table;
}

// Set-up, once per device, with that device current: ask the runtime where this device keeps the array, and put
// the two sigmoid tables (float and double, each at its own offset) into it.  Later calls copy nothing.
int static_scratch_base(StaticScratchSlot **out)
{
   int dev = 0;
   CK(cudaGetDevice(&dev));
   if (dev < 0 || dev >= STATIC_MAX_DEVICES) return FUSEDMM_B200_ERR_LIMIT;
   StaticScratchSlot &slot = g_static_slot[dev];
   if (!slot.base) {
      void *ptr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (e != cudaSuccess || !ptr) {
         fprintf(stderr, "fusedmm_b200: cudaGetSymbolAddress(static scratch) failed on device %d: %s\n", dev,
                 cudaGetErrorString(e));
         cudaGetLastError();
         return FUSEDMM_B200_ERR_CUDA;
      }
      CK(cudaDeviceGetAttribute(&slot.sm_count, cudaDevAttrMultiProcessorCount, dev));
      unsigned char *base = static_cast<unsigned char *>(ptr);
      CK(cudaMemcpy(base + STATIC_OFF_TABLE_F, static_host_sigmoid_table<float>(), SM_TABLE_SIZE * sizeof(float), cudaMemcpyHostToDevice));
      CK(cudaMemcpy(base + STATIC_OFF_TABLE_D, static_host_sigmoid_table<double>(), SM_TABLE_SIZE * sizeof(double), cudaMemcpyHostToDevice));
      slot.base = base;
   }
   *out = &slot;
   return 0;
}

// The row scheduler's four launches on ONE stream (no side stream, no events: creating them allocates),
// with every scratch pointer inside the static array.
template <typename T>
int run_static_scratch(const HostArgs &a, const Decoded &d, const fusedmm_b200_sop &sopk, cudaStream_t user_stream)
{
   constexpr int W = VecOf<T>::W;
   const size_t es = sizeof(T), ps = a.ptr_bits / 8;
   (void)ps;
   const bool need_x = vop_reads_x(d.vop) || rop_reads_x(d.rop);
   const bool need_y = vop_reads_y(d.vop);
   const bool need_val = d.rop == ROP_NOOP && d.vsc != VSC_NOOP;
   if ((need_x && !a.x) || (need_y && (!a.y || !a.indx)) || (need_val && !a.val) || !a.z || !a.pntrb || !a.pntre)
      return FUSEDMM_B200_ERR_ARG;
   if (a.ldz < a.k || (need_x && a.ldx < a.k) || (need_y && a.ldy < a.k)) return FUSEDMM_B200_ERR_ARG;
   const void *arrays[7] = {a.val, a.indx, a.pntrb, a.pntre, a.x, a.y, a.z};
   const bool used[7] = {need_val, need_y, true, true, need_x, need_y, true};
   for (int i = 0; i < 7; i++)
      if (used[i] && !is_device_pointer(arrays[i])) {
         fprintf(stderr, "fusedmm_b200_csr_static_scratch: every array must be in device memory "
                         "(a host array would need a staging buffer, and this entry point allocates nothing)\n");
         return FUSEDMM_B200_ERR_ARG;
      }
   StaticScratchSlot *slot = nullptr;
   CKI(static_scratch_base(&slot));

   Params<T> p;
   memset(&p, 0, sizeof(p));
   p.val = static_cast<const T *>(a.val);
   p.indx = a.indx; p.pntrb = a.pntrb; p.pntre = a.pntre;
   p.x = static_cast<const T *>(a.x); p.y = static_cast<const T *>(a.y); p.z = static_cast<T *>(a.z);
   p.m = a.m; p.k = a.k; p.ldx = a.ldx; p.ldy = a.ldy; p.ldz = a.ldz;
   p.ptr64 = a.ptr_bits == 64; p.idx64 = a.idx_bits == 64;
   p.vop = d.vop; p.rop = d.rop; p.sop = d.sop; p.vsc = d.vsc; p.aop = d.aop;
   p.sop_kind = sopk.kind;
   p.sp0 = static_cast<T>(sopk.p0); p.sp1 = static_cast<T>(sopk.p1); p.sp2 = static_cast<T>(sopk.p2);
   p.accumulate = (t_opt.beta_mode == 0 && d.pattern != PAT_GENERIC) ? (a.beta != 0.0) : 1;
   p.chunk = std::max<int64_t>(512, t_opt.hub_chunk);  // fixed scratch: fewer, longer pieces than the default
   p.counter = reinterpret_cast<unsigned long long *>(slot->base);
   p.hub_row = reinterpret_cast<long long *>(slot->base + STATIC_OFF_HUB_ROW);
   p.hub_base = reinterpret_cast<long long *>(slot->base + STATIC_OFF_HUB_BASE);
   p.hub_cap = STATIC_HUB_CAP;
   p.partials = reinterpret_cast<T *>(slot->base + STATIC_OFF_PARTIALS);
   p.chunk_cap = static_cast<long long>((FUSEDMM_B200_STATIC_SCRATCH_BYTES - STATIC_OFF_PARTIALS) / (static_cast<size_t>(a.k) * es));

   // Sizes beyond the fixed scratch are refused before anything runs.  The bound needs a truthful nnz:
   // a row is split only if it has more than `chunk` edges, so at most nnz/chunk rows are split and they
   // have at most nnz/chunk + (split rows) chunks.
   if (a.nnz < 0) return FUSEDMM_B200_ERR_ARG;
   const long long bound_hubs = a.nnz / p.chunk + 1, bound_chunks = a.nnz / p.chunk + bound_hubs;
   if (bound_hubs > p.hub_cap || bound_chunks > p.chunk_cap) {
      fprintf(stderr, "fusedmm_b200_csr_static_scratch: nnz = %lld with k = %lld needs room for up to %lld split rows and "
                      "%lld partial rows; the %u MiB static scratch holds %lld and %lld. Use fusedmm_b200_csr.\n",
              a.nnz, a.k, bound_hubs, bound_chunks, FUSEDMM_B200_STATIC_SCRATCH_BYTES >> 20, p.hub_cap, p.chunk_cap);
      return FUSEDMM_B200_ERR_LIMIT;
   }

   cudaStream_t st = user_stream ? user_stream : cudaStreamLegacy;  // no stream is created
   if (d.sop == OP_UDEF && sopk.kind == FUSEDMM_SOP_SIGMOID_TABLE_C)  // uploaded once per device at set-up
      p.sop_table = reinterpret_cast<const T *>(slot->base + (sizeof(T) == 4 ? STATIC_OFF_TABLE_F : STATIC_OFF_TABLE_D));
   auto aligned16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
   bool vec_ok = (a.k % W == 0) && (a.ldz % W == 0) && aligned16(p.z) &&
                 (!need_x || ((a.ldx % W == 0) && aligned16(p.x))) && (!need_y || ((a.ldy % W == 0) && aligned16(p.y)));
   int G = 0, NV = 0, U = 0;
   if (vec_ok) {
      choose_tiling(a.k / W, sizeof(T) == 8, &G, &NV, &U);
      if (d.pattern == PAT_GENERIC) tiling_for_generic(G, NV, &U);
      if (G == 0) vec_ok = false;
   }
   const int warps = static_cast<int>(std::min<int64_t>(std::max<int64_t>(t_opt.warps_per_cta, 1), WARPS_PER_CTA));
   const long long rows_per_warp = vec_ok ? 32 / G : 1;
   const long long row_grid = (a.m + warps * rows_per_warp - 1) / (warps * rows_per_warp);
   const long long hub_grid = static_cast<long long>(slot->sm_count) * 8;

   // the array keeps whatever the previous call left in it: the packed counter is the one word that must
   // start at zero (hub list and partial sums are rewritten before they are read)
   CK(cudaMemsetAsync(p.counter, 0, sizeof(unsigned long long), st));
   scan_hub_rows<<<static_cast<unsigned int>((a.m + 255) / 256), 256, 0, st>>>(
      p.pntrb, p.pntre, p.ptr64, p.m, p.chunk, p.counter, p.hub_row, p.hub_base, p.hub_cap);
   // K fills the tiling exactly: the instantiation without bounds predicates, where it is compiled in
   const int Ux = (t_opt.exact_k && static_cast<long long>(G) * NV * W == a.k) ? (U | (1 << 16)) : U;
   p.mode = MODE_HUB_CHUNKS;
   if (vec_ok) { if (!launch_vec<T>(d.pattern, G, NV, Ux, WARPS_PER_CTA, p, hub_grid, st) && !launch_vec<T>(d.pattern, G, NV, U, WARPS_PER_CTA, p, hub_grid, st)) return FUSEDMM_B200_ERR_ARG; }
   else launch_any<T>(p, WARPS_PER_CTA, hub_grid, st);
   launch_fixup<T>(p, static_cast<long long>(slot->sm_count) * 4, st);
   p.mode = MODE_ROWS;
   if (vec_ok) { if (!launch_vec<T>(d.pattern, G, NV, Ux, warps, p, row_grid, st) && !launch_vec<T>(d.pattern, G, NV, U, warps, p, row_grid, st)) return FUSEDMM_B200_ERR_ARG; }
   else launch_any<T>(p, warps, row_grid, st);
   CK(cudaGetLastError());
   long long nh = 0, nchunks = 0;
   slot->async_pending = user_stream != nullptr;
   slot->async_hub_cap = p.hub_cap;
   slot->async_chunk_cap = p.chunk_cap;
   if (!user_stream) {
      unsigned long long packed = 0;
      CK(cudaMemcpyAsync(&packed, p.counter, sizeof(packed), cudaMemcpyDeviceToHost, st));
      CK(cudaStreamSynchronize(st));
      nh = static_cast<long long>(packed >> HUB_SHIFT);
      nchunks = static_cast<long long>(packed & HUB_CHUNK_MASK);
      if (nh > p.hub_cap || nchunks > p.chunk_cap) {  // only possible when nnz understated the edge count
         fprintf(stderr, "fusedmm_b200_csr_static_scratch: the graph has more split rows than nnz allowed for\n");
         return FUSEDMM_B200_ERR_LIMIT;
      }
   }
   memset(&t_info, 0, sizeof(t_info));
   t_info.kernel_launches = 4;
   t_info.pattern = d.pattern;
   t_info.lanes_per_edge = vec_ok ? G : 0;
   t_info.vectors_per_lane = vec_ok ? NV : 0;
   t_info.hub_rows = nh;
   t_info.hub_chunks = nchunks;
   t_info.engine = 1;
   t_info.sop_kind = d.sop == OP_UDEF ? sopk.kind : -1;
   return 0;
}

int32_t letter_to_message(char tkern)
{
   switch (tkern) {
      case 't': return 0x11F55;  // VOP_SUBR | ROP_NORMR | SOP_UDEF | VSC_MUL | AOP_ADD
      case 's': return 0x11F12;  // VOP_COPY_RHS | ROP_DOT | SOP_UDEF | VSC_MUL | AOP_ADD
      case 'm': return 0x11102;  // VOP_COPY_RHS | ROP_NOOP | SOP_COPY | VSC_MUL | AOP_ADD
      case 'g': return 0x10002;  // VOP_COPY_RHS | ROP_NOOP | SOP_NOOP | VSC_NOOP | AOP_ADD
      default: return -1;
   }
}

template <typename PT>
int shard_rows(int64_t m, int32_t nshards, const PT *pntrb, const PT *pntre, int64_t *bounds, int64_t row_weight)
{
   if (m < 0 || nshards < 1 || row_weight < 0 || !bounds || (m > 0 && (!pntrb || !pntre))) return FUSEDMM_B200_ERR_ARG;
   // prefix of the rows' costs (edges + row_weight each), then the first row whose prefix reaches g/nshards of the total
   std::vector<int64_t> pre(m + 1, 0);
   for (int64_t i = 0; i < m; i++)
      pre[i + 1] = pre[i] + row_weight + std::max<int64_t>(0, static_cast<int64_t>(pntre[i]) - static_cast<int64_t>(pntrb[i]));
   const int64_t total = pre[m];
   bounds[0] = 0;
   for (int32_t g = 1; g < nshards; g++) {
      const int64_t target = static_cast<int64_t>((static_cast<__int128>(total) * g) / nshards);
      int64_t r = std::lower_bound(pre.begin(), pre.end(), target) - pre.begin();
      r = std::min<int64_t>(std::max<int64_t>(r, bounds[g - 1]), m);
      bounds[g] = r;
   }
   bounds[nshards] = m;
   return 0;
}

}  // namespace

// =====================================================================================================
// exported symbols
// =====================================================================================================
extern "C" {

int fusedmm_b200_csr(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage, int64_t m,
                     int64_t n, int64_t k, double alpha, int64_t nnz, int64_t rows, int64_t cols,
                     const void *val, const void *indx, const void *pntrb, const void *pntre,
                     const void *x, int64_t ldx, const void *y, int64_t ldy, double beta, void *z,
                     int64_t ldz, const fusedmm_b200_sop *sop, void *stream)
{
   (void)alpha; (void)nnz; (void)rows; (void)cols;  // never read by the reference either (fusedMM.c:487-744)
   return run_call(dtype, ptr_bits, idx_bits, imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, ldx, y, ldy,
                   beta, z, ldz, sop, nullptr, stream);
}

int fusedmm_b200_csr_multi(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage, int64_t m,
                           int64_t n, int64_t k, double alpha, int64_t nnz, int64_t rows, int64_t cols,
                           const void *val, const void *indx, const void *pntrb, const void *pntre,
                           const void *x, int64_t ldx, const void *y, int64_t ldy, double beta, void *z,
                           int64_t ldz, const fusedmm_b200_sop *sop, void *stream, int32_t n_peers,
                           void *const *z_peers, void *z_multicast)
{
   (void)alpha; (void)rows; (void)cols;
   if (n_peers < 0) return FUSEDMM_B200_ERR_ARG;
   return run_call(dtype, ptr_bits, idx_bits, imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, ldx, y, ldy,
                   beta, z, ldz, sop, nullptr, stream, n_peers, z_peers, z_multicast);
}

#define FMM_DEFINE_CSR(NAME, VT, IT, DT, PB, IB)                                                      \
   int NAME(const int32_t imessage, const IT m, const IT n, const IT k, const VT alpha, const IT nnz, \
            const IT rows, const IT cols, const VT *val, const IT *indx, const IT *pntrb,             \
            const IT *pntre, const VT *x, const IT ldx, const VT *y, const IT ldy, const VT beta,     \
            VT *z, const IT ldz)                                                                      \
   {                                                                                                  \
      (void)alpha; (void)nnz; (void)rows; (void)cols;                                                 \
      return run_call(DT, PB, IB, imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, ldx, y, ldy, beta,   \
                      z, ldz, nullptr, nullptr, nullptr);                                             \
   }
FMM_DEFINE_CSR(sfusedMM_csr_i32, float, int32_t, 0, 32, 32)
FMM_DEFINE_CSR(sfusedMM_csr_i64, float, int64_t, 0, 64, 64)
FMM_DEFINE_CSR(dfusedMM_csr_i32, double, int32_t, 1, 32, 32)
FMM_DEFINE_CSR(dfusedMM_csr_i64, double, int64_t, 1, 64, 64)
FMM_DEFINE_CSR(fusedMM_csr, float, int64_t, 0, 64, 64)

#define FMM_DEFINE_CSR_UDEF(NAME, VT, IT, DT, PB, IB)                                                 \
   int NAME(const int32_t imessage, const IT m, const IT n, const IT k, const VT alpha, const IT nnz, \
            const IT rows, const IT cols, const VT *val, const IT *indx, const IT *pntrb,             \
            const IT *pntre, const VT *x, const IT ldx, const VT *y, const IT ldy, const VT beta,     \
            VT *z, const IT ldz, int (*sop_udef)(VT, VT *))                                           \
   {                                                                                                  \
      (void)alpha; (void)nnz; (void)rows; (void)cols;                                                 \
      return run_call(DT, PB, IB, imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, ldx, y, ldy, beta,   \
                      z, ldz, nullptr, reinterpret_cast<void *>(sop_udef), nullptr);                  \
   }
FMM_DEFINE_CSR_UDEF(sfusedMM_csr_i32_udef, float, int32_t, 0, 32, 32)
FMM_DEFINE_CSR_UDEF(sfusedMM_csr_i64_udef, float, int64_t, 0, 64, 64)
FMM_DEFINE_CSR_UDEF(dfusedMM_csr_i32_udef, double, int32_t, 1, 32, 32)
FMM_DEFINE_CSR_UDEF(dfusedMM_csr_i64_udef, double, int64_t, 1, 64, 64)

int sfusedMM_csr_p64i32(const int32_t imessage, const int64_t m, const int64_t n, const int64_t k,
                        const float alpha, const int64_t nnz, const int64_t rows, const int64_t cols,
                        const float *val, const int32_t *indx, const int64_t *pntrb, const int64_t *pntre,
                        const float *x, const int64_t ldx, const float *y, const int64_t ldy,
                        const float beta, float *z, const int64_t ldz)
{
   (void)alpha; (void)nnz; (void)rows; (void)cols;
   return run_call(0, 64, 32, imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz,
                   nullptr, nullptr, nullptr);
}
int dfusedMM_csr_p64i32(const int32_t imessage, const int64_t m, const int64_t n, const int64_t k,
                        const double alpha, const int64_t nnz, const int64_t rows, const int64_t cols,
                        const double *val, const int32_t *indx, const int64_t *pntrb, const int64_t *pntre,
                        const double *x, const int64_t ldx, const double *y, const int64_t ldy,
                        const double beta, double *z, const int64_t ldz)
{
   (void)alpha; (void)nnz; (void)rows; (void)cols;
   return run_call(1, 64, 32, imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz,
                   nullptr, nullptr, nullptr);
}

#define FMM_DEFINE_G(NAME, VT, IT, DT, PB, IB)                                                        \
   void NAME(const char tkern, const IT m, const IT n, const IT k, const VT alpha, const IT nnz,      \
             const IT rows, const IT cols, const VT *val, const IT *indx, const IT *pntrb,            \
             const IT *pntre, const VT *A, const IT lda, const VT *B, const IT ldb, const VT beta,    \
             VT *C, const IT ldc)                                                                     \
   {                                                                                                  \
      (void)alpha; (void)nnz; (void)rows; (void)cols;                                                 \
      const int32_t msg = letter_to_message(tkern);                                                   \
      if (msg < 0) { fprintf(stderr, "Kernel not implemented yet!!!\n"); return; }                    \
      int st = run_call(DT, PB, IB, msg, m, n, k, nnz, val, indx, pntrb, pntre, A, lda, B, ldb, beta, C,   \
                        ldc, nullptr, nullptr, nullptr);                                              \
      if (st) fprintf(stderr, "fusedmm_b200: %s: %s\n", #NAME, fusedmm_b200_status_string(st));      \
   }
FMM_DEFINE_G(sgfusedMM_csr_i32, float, int32_t, 0, 32, 32)
FMM_DEFINE_G(sgfusedMM_csr_i64, float, int64_t, 0, 64, 64)
FMM_DEFINE_G(dgfusedMM_csr_i32, double, int32_t, 1, 32, 32)
FMM_DEFINE_G(dgfusedMM_csr_i64, double, int64_t, 1, 64, 64)

#define FMM_DEFINE_G_UDEF(NAME, VT, IT, DT, PB, IB)                                                   \
   void NAME(const char tkern, const IT m, const IT n, const IT k, const VT alpha, const IT nnz,      \
             const IT rows, const IT cols, const VT *val, const IT *indx, const IT *pntrb,            \
             const IT *pntre, const VT *A, const IT lda, const VT *B, const IT ldb, const VT beta,    \
             VT *C, const IT ldc, int (*sop_udef)(VT, VT *))                                          \
   {                                                                                                  \
      (void)alpha; (void)nnz; (void)rows; (void)cols;                                                 \
      const int32_t msg = letter_to_message(tkern);                                                   \
      if (msg < 0) { fprintf(stderr, "Kernel not implemented yet!!!\n"); return; }                    \
      int st = run_call(DT, PB, IB, msg, m, n, k, nnz, val, indx, pntrb, pntre, A, lda, B, ldb, beta, C,   \
                        ldc, nullptr, reinterpret_cast<void *>(sop_udef), nullptr);                   \
      if (st) fprintf(stderr, "fusedmm_b200: %s: %s\n", #NAME, fusedmm_b200_status_string(st));      \
   }
FMM_DEFINE_G_UDEF(sgfusedMM_csr_i32_udef, float, int32_t, 0, 32, 32)
FMM_DEFINE_G_UDEF(sgfusedMM_csr_i64_udef, float, int64_t, 0, 64, 64)
FMM_DEFINE_G_UDEF(dgfusedMM_csr_i32_udef, double, int32_t, 1, 32, 32)
FMM_DEFINE_G_UDEF(dgfusedMM_csr_i64_udef, double, int64_t, 1, 64, 64)

int fusedmm_b200_zero_empty_rows(int32_t dtype, int32_t ptr_bits, int64_t m, int64_t k, const void *pntrb,
                                 const void *pntre, void *z, int64_t ldz, void *stream)
{
   if ((dtype != 0 && dtype != 1) || (ptr_bits != 32 && ptr_bits != 64) || m < 0 || k < 0 || ldz < k) return FUSEDMM_B200_ERR_ARG;
   if (m == 0 || k == 0) return 0;
   if (!pntrb || !pntre || !z) return FUSEDMM_B200_ERR_ARG;
   if (!is_device_pointer(pntrb) || !is_device_pointer(pntre) || !is_device_pointer(z)) return FUSEDMM_B200_ERR_ARG;
   cudaStream_t st = static_cast<cudaStream_t>(stream);
   const unsigned int grid = static_cast<unsigned int>((m + 255) / 256);
   if (dtype == 0) zero_empty_rows_kernel<float><<<grid, 256, 0, st>>>(pntrb, pntre, ptr_bits == 64, m, k, static_cast<float *>(z), ldz);
   else zero_empty_rows_kernel<double><<<grid, 256, 0, st>>>(pntrb, pntre, ptr_bits == 64, m, k, static_cast<double *>(z), ldz);
   CK(cudaGetLastError());
   if (!stream) CK(cudaStreamSynchronize(st));
   return 0;
}

int fusedmm_b200_jit_prepare(int32_t dtype, int32_t imessage, int64_t k)
{
   {
      std::lock_guard<std::mutex> lock(g_mu);
      t_opt = g_opt;
   }
   if ((dtype != 0 && dtype != 1) || k <= 0) return FUSEDMM_B200_ERR_ARG;
   Decoded d;
   int st = decode_message(imessage, t_opt, &d);
   if (st) return st;
   if (d.pattern != PAT_GENERIC || d.aop == AOP_NOOP) return 0;  // built in, or nothing to compute
   const int W = dtype == 0 ? 4 : 2;
   if (k % W != 0) return 0;                                      // the element-strided kernels take it
   int G = 0, NV = 0, U = 0;
   choose_tiling(k / W, dtype == 1, &G, &NV, &U);
   if (G == 0) return 0;
   return jit_prepare(dtype, d.vop, d.rop, d.vsc, d.aop, G, NV, U & 0xFF, jit_budget(G, NV, U & 0xFF, U >> 8), 0) == 0 ? 0 : FUSEDMM_B200_ERR_NO_OPT;
}

int fusedmm_b200_jit_stats(int64_t *out)
{
   if (!out) return FUSEDMM_B200_ERR_ARG;
   const JitStats s = jit_stats();
   out[0] = s.compiled; out[1] = s.disk_hits; out[2] = s.launches; out[3] = s.failures; out[4] = s.nvrtc_found;
   return 0;
}

int fusedmm_b200_set_sop(int32_t kind, double p0, double p1, double p2)
{
   if (kind < 0 || kind >= FUSEDMM_SOP_KIND_COUNT) return FUSEDMM_B200_ERR_ARG;
   std::lock_guard<std::mutex> lock(g_mu);
   g_sop.kind = kind; g_sop.reserved = 0; g_sop.p0 = p0; g_sop.p1 = p1; g_sop.p2 = p2;
   return 0;
}
int fusedmm_b200_get_sop(fusedmm_b200_sop *out)
{
   if (!out) return FUSEDMM_B200_ERR_ARG;
   std::lock_guard<std::mutex> lock(g_mu);
   *out = g_sop;
   return 0;
}

int fusedmm_b200_csr_static_scratch(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage, int64_t m,
                                    int64_t n, int64_t k, double alpha, int64_t nnz, int64_t rows, int64_t cols,
                                    const void *val, const void *indx, const void *pntrb, const void *pntre,
                                    const void *x, int64_t ldx, const void *y, int64_t ldy, double beta, void *z,
                                    int64_t ldz, const fusedmm_b200_sop *sop, void *stream)
{
   (void)alpha; (void)rows; (void)cols;
   if ((dtype != 0 && dtype != 1) || (ptr_bits != 32 && ptr_bits != 64) || (idx_bits != 32 && idx_bits != 64))
      return FUSEDMM_B200_ERR_ARG;
   fusedmm_b200_sop sopk;
   {
      std::lock_guard<std::mutex> lock(g_mu);
      t_opt = g_opt;
      sopk = g_sop;
   }
   // the array is per device: one call at a time per device (no context is created: that would allocate)
   int dev = 0;
   CK(cudaGetDevice(&dev));
   if (dev < 0 || dev >= MAX_DEVICES) return FUSEDMM_B200_ERR_LIMIT;
   std::lock_guard<std::mutex> device_lock(g_ctx[dev].mu);
   Decoded d;
   int st = decode_message(imessage, t_opt, &d);
   if (st) return st;
   if (d.sop == OP_UDEF && sop) {
      if (sop->kind < 0 || sop->kind >= FUSEDMM_SOP_KIND_COUNT) return FUSEDMM_B200_ERR_UDEF;
      sopk = *sop;
   }
   if (m < 0 || k < 0) return FUSEDMM_B200_ERR_ARG;
   if (d.aop == AOP_NOOP || m == 0 || k == 0) return 0;
   HostArgs a = {imessage, m, n, k, nnz, val, indx, pntrb, pntre, x, y, z, ldx, ldy, ldz, beta, ptr_bits, idx_bits, 0, nullptr, nullptr, nullptr};
   return dtype == 0 ? run_static_scratch<float>(a, d, sopk, static_cast<cudaStream_t>(stream))
                     : run_static_scratch<double>(a, d, sopk, static_cast<cudaStream_t>(stream));
}

int fusedmm_b200_plan_create(int32_t ptr_bits, int32_t idx_bits, int64_t m, int64_t nnz, const void *indx,
                             const void *pntrb, const void *pntre, int32_t val_dtype, const void *val,
                             fusedmm_b200_plan **out)
{
   (void)nnz;
   if (!out || m < 0 || (ptr_bits != 32 && ptr_bits != 64) || (idx_bits != 32 && idx_bits != 64) ||
       (val && val_dtype != 0 && val_dtype != 1) || (m > 0 && (!pntrb || !pntre)))
      return FUSEDMM_B200_ERR_ARG;
   *out = nullptr;
   DeviceCtx *c = nullptr;
   std::unique_lock<std::mutex> device_lock;
   CKI(enter_device(&c, &device_lock));
   CK(cudaDeviceSynchronize());
   fusedmm_b200_plan *pl = new fusedmm_b200_plan();
   pl->device = c->device;
   pl->ptr_bits = ptr_bits; pl->idx_bits = idx_bits; pl->val_dtype = val ? val_dtype : -1; pl->m = m;
   const size_t ps = ptr_bits / 8, is = idx_bits / 8, vs = val_dtype == 1 ? 8 : 4;
   auto fail = [&](int st) { fusedmm_b200_plan_destroy(pl); return st; };
   // the edge extent of the arrays: largest row end
   long long ext = 0;
   if (m > 0) {
      std::vector<char> tmp;
      const void *hpe = pntre;
      if (is_device_pointer(pntre)) {
         tmp.resize(m * ps);
         if (cudaMemcpy(tmp.data(), pntre, m * ps, cudaMemcpyDeviceToHost) != cudaSuccess) return fail(FUSEDMM_B200_ERR_CUDA);
         hpe = tmp.data();
      }
      ext = ptr_bits == 64 ? max_entry(static_cast<const int64_t *>(hpe), m) : max_entry(static_cast<const int32_t *>(hpe), m);
   }
   pl->nnz = ext;
   const void *src[4] = {val, indx, pntrb, pntre};
   const size_t bytes[4] = {static_cast<size_t>(ext) * vs, static_cast<size_t>(ext) * is, static_cast<size_t>(m) * ps, static_cast<size_t>(m) * ps};
   const void **dst[4] = {&pl->val, &pl->indx, &pl->pntrb, &pl->pntre};
   const bool pe_is_pb1 = pntrb && static_cast<const char *>(pntre) == static_cast<const char *>(pntrb) + ps;
   for (int i = 0; i < 4; i++) {
      if (!src[i]) continue;
      if (is_device_pointer(src[i])) { *dst[i] = src[i]; continue; }  // borrowed: the caller keeps it alive
      if (i == 3 && pe_is_pb1 && pl->own[2]) { pl->pntre = static_cast<const char *>(pl->own[2]) + ps; continue; }
      const size_t nb = (i == 2 && pe_is_pb1) ? bytes[i] + ps : bytes[i];  // (rowptr, rowptr+1): one copy of m+1 entries
      if (cudaMalloc(&pl->own[i], std::max<size_t>(nb, 16)) != cudaSuccess) { cudaGetLastError(); return fail(FUSEDMM_B200_ERR_NOMEM); }
      if (nb && cudaMemcpy(pl->own[i], src[i], nb, cudaMemcpyHostToDevice) != cudaSuccess) return fail(FUSEDMM_B200_ERR_CUDA);
      *dst[i] = pl->own[i];
   }
   // split-row list, sized by its upper bound so that the scan cannot overflow it
   pl->chunk = std::max<int64_t>(32, t_opt.hub_chunk);
   if (ext > 0 && ext < (1ll << 24)) pl->chunk = std::min<long long>(pl->chunk, 128);  // as in a plain call; K is not known yet
   if (ext > 0 && ext < (1ll << 21)) pl->chunk = std::min<long long>(pl->chunk, 64);
   const long long cap = ext / pl->chunk + 1;
   if (cudaMalloc(&pl->hub_row, cap * sizeof(long long)) != cudaSuccess || cudaMalloc(&pl->hub_base, cap * sizeof(long long)) != cudaSuccess ||
       cudaMalloc(&pl->counter, 256) != cudaSuccess) { cudaGetLastError(); return fail(FUSEDMM_B200_ERR_NOMEM); }
   if (cudaMemset(pl->counter, 0, 256) != cudaSuccess) return fail(FUSEDMM_B200_ERR_CUDA);
   if (m > 0) {
      scan_hub_rows<<<static_cast<unsigned int>((m + 255) / 256), 256, 0, c->stream>>>(pl->pntrb, pl->pntre, ptr_bits == 64, m, pl->chunk,
                                                                                     pl->counter, pl->hub_row, pl->hub_base, cap);
      unsigned long long packed = 0;
      if (cudaMemcpyAsync(&packed, pl->counter, sizeof(packed), cudaMemcpyDeviceToHost, c->stream) != cudaSuccess ||
          cudaStreamSynchronize(c->stream) != cudaSuccess) return fail(FUSEDMM_B200_ERR_CUDA);
      pl->nh = static_cast<long long>(packed >> HUB_SHIFT);
      pl->nchunks = static_cast<long long>(packed & HUB_CHUNK_MASK);
      if (t_opt.row_bins != 0 && m < (1ll << 32) && (t_opt.row_bins == 2 || ext >= (1ll << 22))) {
         if (cudaMalloc(&pl->row_order, m * sizeof(unsigned int)) != cudaSuccess) { cudaGetLastError(); return fail(FUSEDMM_B200_ERR_NOMEM); }
         bin_rows_kernel<<<static_cast<unsigned int>((m + ROW_BIN_TILE - 1) / ROW_BIN_TILE), 256, 0, c->stream>>>(
            pl->pntrb, pl->pntre, ptr_bits == 64, m, pl->chunk, pl->row_order);
         if (cudaStreamSynchronize(c->stream) != cudaSuccess) return fail(FUSEDMM_B200_ERR_CUDA);
      }
      // the visiting order of the chunks is made once here; the column count is not an argument of a plan: the largest
      // first column id of a chunk stands in for it
      if (pl->indx && ((t_opt.chunk_order == 1 && pl->nchunks >= 1024) || (t_opt.chunk_order == 2 && pl->nchunks > 0))) {
         unsigned int *cnt = nullptr;
         if (cudaMalloc(&pl->order, pl->nchunks * sizeof(long long)) != cudaSuccess || cudaMalloc(&cnt, 3 * ORDER_BUCKETS * sizeof(unsigned int)) != cudaSuccess) {
            cudaGetLastError();
            if (cnt) cudaFree(cnt);
            return fail(FUSEDMM_B200_ERR_NOMEM);
         }
         unsigned long long top = 0;
         bool ok = cudaMemsetAsync(cnt, 0, sizeof(unsigned long long), c->stream) == cudaSuccess;
         if (ok) order_chunks_kernel<<<static_cast<unsigned int>(c->sm_count * 8), 256, 0, c->stream>>>(
            2, pl->pntrb, pl->pntre, ptr_bits == 64, pl->indx, idx_bits == 64, 0, pl->chunk, pl->counter, pl->hub_row, pl->hub_base, cap,
            pl->nchunks, cnt, nullptr, nullptr);
         ok = ok && cudaMemcpyAsync(&top, cnt, sizeof(top), cudaMemcpyDeviceToHost, c->stream) == cudaSuccess &&
              cudaStreamSynchronize(c->stream) == cudaSuccess;
         ok = ok && enqueue_chunk_order(pl->pntrb, pl->pntre, ptr_bits == 64, pl->indx, idx_bits == 64, static_cast<long long>(std::max<unsigned long long>(top, 1)),
                                        pl->chunk, pl->counter, pl->hub_row, pl->hub_base, cap, pl->nchunks, cnt, pl->order, c->sm_count,
                                        c->stream) == cudaSuccess;
         ok = ok && cudaStreamSynchronize(c->stream) == cudaSuccess;
         cudaFree(cnt);
         if (!ok) return fail(FUSEDMM_B200_ERR_CUDA);
      }
   }
   *out = pl;
   return 0;
}

int fusedmm_b200_plan_csr(const fusedmm_b200_plan *plan, int32_t dtype, int32_t imessage, int64_t n, int64_t k,
                          const void *x, int64_t ldx, const void *y, int64_t ldy, double beta, void *z, int64_t ldz,
                          const fusedmm_b200_sop *sop, void *stream)
{
   if (!plan) return FUSEDMM_B200_ERR_ARG;
   int dev = -1;
   if (cudaGetDevice(&dev) != cudaSuccess || dev != plan->device) return FUSEDMM_B200_ERR_ARG;
   const bool uses_val = ((imessage >> 4) & 0xF) == 0 && ((imessage >> 12) & 0xF) != 0;
   if (uses_val && plan->val_dtype != dtype) return FUSEDMM_B200_ERR_ARG;  // edge values of the other type, or none
   return run_call(dtype, plan->ptr_bits, plan->idx_bits, imessage, plan->m, n, k, plan->nnz, plan->val, plan->indx,
                   plan->pntrb, plan->pntre, x, ldx, y, ldy, beta, z, ldz, sop, nullptr, stream, 0, nullptr, nullptr, plan);
}

int fusedmm_b200_plan_destroy(fusedmm_b200_plan *plan)
{
   if (!plan) return 0;
   cudaDeviceSynchronize();
   for (void *q : plan->own) if (q) cudaFree(q);
   if (plan->hub_row) cudaFree(plan->hub_row);
   if (plan->hub_base) cudaFree(plan->hub_base);
   if (plan->order) cudaFree(plan->order);
   if (plan->row_order) cudaFree(plan->row_order);
   if (plan->counter) cudaFree(plan->counter);
   delete plan;
   return 0;
}

int fusedmm_b200_stream_status(void)
{
   int cur_dev = -1;
   if (cudaGetDevice(&cur_dev) != cudaSuccess || cur_dev < 0 || cur_dev >= MAX_DEVICES) { cudaGetLastError(); return FUSEDMM_B200_ERR_CUDA; }
   std::unique_lock<std::mutex> device_lock(g_ctx[cur_dev].mu);
   {  // a call of the entry point that allocates nothing, enqueued on a caller's stream (nothing is allocated here either)
      if (g_static_slot[cur_dev].base && g_static_slot[cur_dev].async_pending) {
         StaticScratchSlot &slot = g_static_slot[cur_dev];
         unsigned long long packed = 0;
         CK(cudaMemcpy(&packed, slot.base, sizeof(packed), cudaMemcpyDeviceToHost));
         slot.async_pending = false;
         if (static_cast<long long>(packed >> HUB_SHIFT) > slot.async_hub_cap ||
             static_cast<long long>(packed & HUB_CHUNK_MASK) > slot.async_chunk_cap)
            return FUSEDMM_B200_ERR_LIMIT;  // nnz understated the graph: the split rows of that call were not computed
      }
   }
   DeviceCtx *c = &g_ctx[cur_dev];
   if (!c->ready || !c->async_pending) return 0;
   unsigned long long words[2] = {0, 0};
   CK(cudaMemcpy(words, c->counter.ptr, sizeof(words), cudaMemcpyDeviceToHost));
   c->async_pending = false;
   if (c->async_engine == 2) {
      const long long nq = static_cast<long long>(words[1]);
      const long long cap = std::min<long long>(c->part_cap, static_cast<long long>(c->heads.bytes / (static_cast<size_t>(c->async_k) * c->async_elt)));
      if (nq <= cap) return 0;
      c->part_cap = nq + nq / 16 + 64;
      CKI(ensure_buf(c->part, (c->part_cap + 1) * sizeof(long long)));
      CKI(ensure_buf(c->heads, static_cast<size_t>(c->part_cap) * c->async_k * c->async_elt));
      return FUSEDMM_B200_ERR_LIMIT;
   }
   const unsigned long long packed = words[0];
   const long long nh = static_cast<long long>(packed >> HUB_SHIFT);
   const long long nchunks = static_cast<long long>(packed & HUB_CHUNK_MASK);
   const long long cap = static_cast<long long>(c->partials.bytes / (static_cast<size_t>(c->async_k) * c->async_elt));
   if (nh <= c->hub_cap && nchunks <= cap) return 0;
   if (nh > c->hub_cap) {
      c->hub_cap = nh + nh / 4 + 1024;
      CKI(ensure_buf(c->hub_row, c->hub_cap * sizeof(long long)));
      CKI(ensure_buf(c->hub_base, c->hub_cap * sizeof(long long)));
   }
   if (nchunks > cap) CKI(ensure_buf(c->partials, static_cast<size_t>(nchunks + nchunks / 8 + 64) * c->async_k * c->async_elt));
   return FUSEDMM_B200_ERR_LIMIT;
}

int fusedmm_b200_check_csr(int32_t ptr_bits, int32_t idx_bits, int64_t m, int64_t n, const void *indx,
                           const void *pntrb, const void *pntre, int64_t *report)
{
   if ((ptr_bits != 32 && ptr_bits != 64) || (idx_bits != 32 && idx_bits != 64) || m < 0 || !report) return FUSEDMM_B200_ERR_ARG;
   for (int i = 0; i < 4; i++) report[i] = 0;
   if (m == 0) return 0;
   if (!pntrb || !pntre || !indx) return FUSEDMM_B200_ERR_ARG;
   DeviceCtx *c = nullptr;
   std::unique_lock<std::mutex> device_lock;
   CKI(enter_device(&c, &device_lock));
   const size_t ps = ptr_bits / 8, is = idx_bits / 8;
   const void *dpb = pntrb, *dpe = pntre, *dix = indx;
   CK(cudaDeviceSynchronize());
   if (!is_device_pointer(pntrb)) {
      CKI(ensure_buf(c->stage[2], m * ps));
      CK(cudaMemcpyAsync(c->stage[2].ptr, pntrb, m * ps, cudaMemcpyHostToDevice, c->stream));
      dpb = c->stage[2].ptr;
   }
   if (!is_device_pointer(pntre)) {
      CKI(ensure_buf(c->stage[3], m * ps));
      CK(cudaMemcpyAsync(c->stage[3].ptr, pntre, m * ps, cudaMemcpyHostToDevice, c->stream));
      dpe = c->stage[3].ptr;
   }
   if (!is_device_pointer(indx)) {
      std::vector<char> tmp;
      const void *hpe = pntre;
      if (is_device_pointer(pntre)) {
         tmp.resize(m * ps);
         CK(cudaMemcpy(tmp.data(), pntre, m * ps, cudaMemcpyDeviceToHost));
         hpe = tmp.data();
      }
      const long long ext = ptr_bits == 64 ? max_entry(static_cast<const int64_t *>(hpe), m) : max_entry(static_cast<const int32_t *>(hpe), m);
      CKI(ensure_buf(c->stage[1], std::max<long long>(ext, 1) * is));
      CK(cudaMemcpyAsync(c->stage[1].ptr, indx, ext * is, cudaMemcpyHostToDevice, c->stream));
      dix = c->stage[1].ptr;
   }
   unsigned long long *rep = static_cast<unsigned long long *>(c->counter.ptr) + 16;  // words 16..19 of the counter block
   CK(cudaMemsetAsync(rep, 0, 4 * sizeof(unsigned long long), c->stream));
   check_csr_kernel<<<c->sm_count * 8, 256, 0, c->stream>>>(dpb, dpe, dix, ptr_bits == 64, idx_bits == 64, m, n, rep);
   CK(cudaGetLastError());
   unsigned long long host[4] = {0, 0, 0, 0};
   CK(cudaMemcpyAsync(host, rep, sizeof(host), cudaMemcpyDeviceToHost, c->stream));
   CK(cudaStreamSynchronize(c->stream));
   for (int i = 0; i < 4; i++) report[i] = static_cast<int64_t>(host[i]);
   return (host[0] || host[1]) ? FUSEDMM_B200_ERR_ARG : 0;
}

int fusedmm_b200_shard_rows_i32(int64_t m, int32_t nshards, const int32_t *pntrb, const int32_t *pntre, int64_t *bounds)
{
   return shard_rows(m, nshards, pntrb, pntre, bounds);
}
int fusedmm_b200_shard_rows_i64(int64_t m, int32_t nshards, const int64_t *pntrb, const int64_t *pntre, int64_t *bounds)
{
   return shard_rows(m, nshards, pntrb, pntre, bounds);
}
int fusedmm_b200_shard_rows_weighted_i32(int64_t m, int32_t nshards, const int32_t *pntrb, const int32_t *pntre, int64_t row_weight,
                                         int64_t *bounds)
{
   return shard_rows(m, nshards, pntrb, pntre, bounds, row_weight);
}
int fusedmm_b200_shard_rows_weighted_i64(int64_t m, int32_t nshards, const int64_t *pntrb, const int64_t *pntre, int64_t row_weight,
                                         int64_t *bounds)
{
   return shard_rows(m, nshards, pntrb, pntre, bounds, row_weight);
}

static int64_t *option_slot(const char *name)
{
   if (!name) return nullptr;
   if (!strcmp(name, "beta_mode")) return &g_opt.beta_mode;
   if (!strcmp(name, "accept_vop_noop")) return &g_opt.accept_vop_noop;
   if (!strcmp(name, "hub_chunk")) return &g_opt.hub_chunk;
   if (!strcmp(name, "force_tiling")) return &g_opt.force_tiling;
   if (!strcmp(name, "force_generic")) return &g_opt.force_generic;
   if (!strcmp(name, "warps_per_cta")) return &g_opt.warps_per_cta;
   if (!strcmp(name, "engine")) return &g_opt.engine;
   if (!strcmp(name, "edge_quantum")) return &g_opt.edge_quantum;
   if (!strcmp(name, "stream_depth")) return &g_opt.stream_depth;
   if (!strcmp(name, "side_priority")) return &g_opt.side_priority;
   if (!strcmp(name, "side_stream")) return &g_opt.side_stream;
   if (!strcmp(name, "force_tiling_rows")) return &g_opt.force_tiling_rows;
   if (!strcmp(name, "chunk_ctas_per_sm")) return &g_opt.chunk_ctas_per_sm;
   if (!strcmp(name, "chunk_order")) return &g_opt.chunk_order;
   if (!strcmp(name, "row_bins")) return &g_opt.row_bins;
   if (!strcmp(name, "blocked_inputs")) return &g_opt.blocked_inputs;
   if (!strcmp(name, "strict_udef")) return &g_opt.strict_udef;
   if (!strcmp(name, "multi_skip_empty_rows")) return &g_opt.multi_skip_empty_rows;
   if (!strcmp(name, "jit")) return &g_opt.jit;
   if (!strcmp(name, "pdl")) return &g_opt.pdl;
   if (!strcmp(name, "jit_call_shape")) return &g_opt.jit_call_shape;
   if (!strcmp(name, "offset32")) return &g_opt.offset32;
   if (!strcmp(name, "hub_cap_initial")) return &g_opt.hub_cap_initial;
   if (!strcmp(name, "jit_shape_mask")) return &g_opt.jit_shape_mask;
   if (!strcmp(name, "exact_k")) return &g_opt.exact_k;
   if (!strcmp(name, "element_vectors")) return &g_opt.element_vectors;
   if (!strcmp(name, "bulk_chunks")) return &g_opt.bulk_chunks;
   if (!strcmp(name, "bulk_warps")) return &g_opt.bulk_warps;
   if (!strcmp(name, "bulk_ctas_per_sm")) return &g_opt.bulk_ctas_per_sm;
   if (!strcmp(name, "timing_detail")) return &g_opt.timing_detail;
   if (!strcmp(name, "inject_alloc_failure")) return &g_fail_alloc_in;
   return nullptr;
}
// FUSEDMM_B200_OPTIONS="name=value,name=value": options set from the environment when the library is loaded, for
// programs that cannot be changed to call fusedmm_b200_set_option (unknown names and malformed items are ignored).
static struct EnvOptions {
   EnvOptions()
   {
      const char *e = getenv("FUSEDMM_B200_OPTIONS");
      if (!e) return;
      std::string all(e);
      size_t pos = 0;
      while (pos < all.size()) {
         size_t end = all.find(',', pos);
         if (end == std::string::npos) end = all.size();
         const std::string item = all.substr(pos, end - pos);
         const size_t eq = item.find('=');
         if (eq != std::string::npos) {
            int64_t *slot = option_slot(item.substr(0, eq).c_str());
            char *rest = nullptr;
            const long long v = strtoll(item.c_str() + eq + 1, &rest, 10);
            if (slot && rest && *rest == '\0' && v >= 0) *slot = v;
         }
         pos = end + 1;
      }
   }
} g_env_options;

int fusedmm_b200_set_option(const char *name, int64_t value)
{
   std::lock_guard<std::mutex> lock(g_mu);
   int64_t *s = option_slot(name);
   if (!s || value < 0) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.force_generic && value > 2) return FUSEDMM_B200_ERR_ARG;
   if ((s == &g_opt.beta_mode || s == &g_opt.accept_vop_noop || s == &g_opt.side_priority || s == &g_opt.strict_udef || s == &g_opt.multi_skip_empty_rows || s == &g_opt.pdl || s == &g_opt.timing_detail || s == &g_opt.exact_k || s == &g_opt.element_vectors) && value > 1) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.bulk_chunks && value != 0 && value != 16 && value != 32) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.bulk_warps && (value < 1 || value > WARPS_PER_CTA)) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.hub_chunk && (value < 32 || value > (1ll << 30))) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.warps_per_cta && (value < 1 || value > WARPS_PER_CTA)) return FUSEDMM_B200_ERR_ARG;
   if ((s == &g_opt.engine || s == &g_opt.jit || s == &g_opt.jit_call_shape) && value > 2) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.chunk_ctas_per_sm && (value < 1 || value > 64)) return FUSEDMM_B200_ERR_ARG;
   if ((s == &g_opt.chunk_order || s == &g_opt.row_bins) && (value < 0 || value > 2)) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.edge_quantum && (value < 32 || value > (1ll << 24))) return FUSEDMM_B200_ERR_ARG;
   if (s == &g_opt.stream_depth && (value < 1 || value > 32)) return FUSEDMM_B200_ERR_ARG;
   *s = value;
   return 0;
}
int fusedmm_b200_get_option(const char *name, int64_t *value)
{
   std::lock_guard<std::mutex> lock(g_mu);
   int64_t *s = option_slot(name);
   if (!s || !value) return FUSEDMM_B200_ERR_ARG;
   *value = *s;
   return 0;
}

int fusedmm_b200_last_call_info(fusedmm_b200_call_info *out)
{
   if (!out) return FUSEDMM_B200_ERR_ARG;
   *out = t_info;
   return 0;
}

const char *fusedmm_b200_status_string(int status)
{
   switch (status) {
      case FUSEDMM_B200_OK: return "success";
      case FUSEDMM_B200_ERR_VOP: return "unknown VOP code";
      case FUSEDMM_B200_ERR_ROP: return "unknown ROP code";
      case FUSEDMM_B200_ERR_AOP: return "unknown AOP code";
      case FUSEDMM_B200_ERR_SOP: return "unknown SOP code";
      case FUSEDMM_B200_ERR_VSC: return "unknown VSC code";
      case FUSEDMM_B200_ERR_NOMEM: return "out of device memory";
      case FUSEDMM_B200_ERR_UDEF: return "user-defined function has no device implementation";
      case FUSEDMM_B200_ERR_NO_OPT: return "no optimised implementation";
      case FUSEDMM_B200_ERR_CUDA: return "CUDA error or no usable device";
      case FUSEDMM_B200_ERR_ARG: return "invalid argument";
      case FUSEDMM_B200_ERR_LIMIT: return "capacity exceeded";
      default: return "unknown status";
   }
}
const char *fusedmm_b200_version(void) { return "fusedmm_b200 0.1 (sm_100a)"; }

int fusedmm_b200_release(void)
{
   std::lock_guard<std::mutex> lock(g_mu);
   int cur = 0;
   if (cudaGetDevice(&cur) != cudaSuccess) { cudaGetLastError(); return FUSEDMM_B200_ERR_CUDA; }
   for (DeviceCtx &c : g_ctx) {
      if (!c.ready) continue;
      std::lock_guard<std::mutex> device_lock(c.mu);
      cudaSetDevice(c.device);
      cudaStreamSynchronize(c.stream);
      DevBuf *bufs[] = {&c.stage[0], &c.stage[1], &c.stage[2], &c.stage[3], &c.stage[4], &c.stage[5], &c.stage[6],
                        &c.hub_row, &c.hub_base, &c.partials, &c.order, &c.order_cnt, &c.row_order, &c.table_f, &c.table_d, &c.part, &c.heads};
      for (DevBuf *b : bufs) { if (b->ptr) cudaFree(b->ptr); b->ptr = nullptr; b->bytes = 0; }
      c.hub_cap = 0;
      c.part_cap = 0;
   }
   cudaSetDevice(cur);
   return 0;
}

}  // extern "C"
