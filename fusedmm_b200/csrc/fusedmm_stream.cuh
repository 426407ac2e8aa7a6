// fusedmm_stream.cuh -- the edge-stream scheduler: nnz-split with row splitting, no atomics.
//
// Needs the usual CSR layout in which row r+1 starts where row r ends (pntre == pntrb + 1 entry,
// which is how every caller of the reference passes it: fusedMMtime.cpp:1437, "rowptr, rowptr+1").
// The edges [E0, E1) of the m rows are one contiguous stream, cut into quanta of Q edges.  A "virtual
// warp" (G lanes; a warp holds 32/G of them) owns one quantum at a time and walks through it edge by
// edge with U neighbour-row gathers in flight, crossing row boundaries without draining: when the
// edge position passes the end of the current row the accumulator is stored and the next row's X_u
// (fetched one row ahead) takes over.  Every quantum is the same amount of gather work whatever the
// degree distribution, so a persistent grid needs no dynamic balancing and rows of any length (hub
// rows of power-law graphs included) need no special path:
//   * a row that lies inside one quantum is written to Z directly;
//   * a row that starts in quantum w and continues: its first piece is written to Z directly;
//   * the piece of a row that started in an earlier quantum goes to heads[w] (at most one per
//     quantum), and stream_fixup_kernel adds heads[w], heads[w+1], ... to Z[row] in quantum order
//     after the main kernel, which makes the result independent of scheduling.
// This replaces the reference's row scheduler (fusedMM.c:633-676: contiguous row ranges per OpenMP
// thread, rows never split, recomputed by every thread on every call).
#pragma once
#include "fusedmm_kernels.cuh"

namespace fmm {

constexpr long long POS_INF_LL = 0x7fffffffffffffffLL;

// ---- cp.async (global -> shared, 16 bytes, cached in L2 only) and its per-thread group bookkeeping ----
__device__ __forceinline__ void cp_async_16(unsigned smem_addr, const void *gptr)
{
   asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most n of this thread's most recent groups are still in flight; n is rounded down to
// one of the values that have a case here (waiting for more than asked is always correct)
__device__ __forceinline__ void cp_async_wait_pending(unsigned n)
{
   if (n >= 28) asm volatile("cp.async.wait_group 28;" ::: "memory");
   else if (n >= 24) asm volatile("cp.async.wait_group 24;" ::: "memory");
   else if (n >= 16) asm volatile("cp.async.wait_group 16;" ::: "memory");
   else if (n >= 12) asm volatile("cp.async.wait_group 12;" ::: "memory");
   else if (n >= 8) asm volatile("cp.async.wait_group 8;" ::: "memory");
   else if (n >= 4) asm volatile("cp.async.wait_group 4;" ::: "memory");
   else asm volatile("cp.async.wait_group 0;" ::: "memory");
}
template <typename T>
__device__ __forceinline__ void ld_shared_vec(unsigned smem_addr, T (&out)[VecOf<T>::W]);
template <>
__device__ __forceinline__ void ld_shared_vec<float>(unsigned smem_addr, float (&out)[4])
{
   asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3]) : "r"(smem_addr) : "memory");
}
template <>
__device__ __forceinline__ void ld_shared_vec<double>(unsigned smem_addr, double (&out)[2])
{
   asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];" : "=d"(out[0]), "=d"(out[1]) : "r"(smem_addr) : "memory");
}

struct StreamShape {
   long long e0, e1, nq;  // first edge, one past the last edge, number of quanta
};
template <typename T>
__device__ __forceinline__ StreamShape stream_shape(const Params<T> &p)
{
   StreamShape s;
   s.e0 = ld_index(p.pntrb, 0, p.ptr64);
   s.e1 = ld_index(p.pntre, p.m - 1, p.ptr64);
   const long long tot = s.e1 > s.e0 ? s.e1 - s.e0 : 0;
   s.nq = tot == 0 ? 1 : (tot + p.quantum - 1) / p.quantum;
   return s;
}

// Pass 1 (one launch, two grid-stride loops):
//  (a) part[w] = first row r with pntre[r] > E0 + w*Q, i.e. the row that holds the first edge of
//      quantum w, by binary search;  (b) rows without edges are set to 0 when Z is overwritten.
// counter[1] receives the number of quanta so that the host can see whether the scratch was big enough.
template <typename T>
__global__ void __launch_bounds__(256) stream_partition_kernel(const Params<T> p)
{
   const StreamShape sh = stream_shape(p);
   const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
   const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
   if (tid == 0) p.counter[1] = static_cast<unsigned long long>(sh.nq);
   if (sh.nq <= p.part_cap) {
      for (long long w = tid; w <= sh.nq; w += nthreads) {
         const long long a = sh.e0 + w * p.quantum;
         long long lo = 0, hi = p.m;  // first r in [0, m] with pntre[r] > a
         while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if (ld_index(p.pntre, mid, p.ptr64) > a) hi = mid; else lo = mid + 1;
         }
         p.part[w] = lo;
      }
   }
   if (!p.accumulate) {
      // a row without edges gets zeros (what the reference's optimised kernels store for it,
      // kernels/codegen/genkern.base:287-295 and :577-581): each lane tests one row, the warp then
      // fills the rows that were found together
      const int lane = threadIdx.x & 31;
      const long long nwarps = nthreads >> 5;
      for (long long base = (tid >> 5) * 32; base < p.m; base += nwarps * 32) {
         const long long r = base + lane;
         const bool empty = r < p.m && ld_index(p.pntre, r, p.ptr64) <= ld_index(p.pntrb, r, p.ptr64);
         unsigned mask = __ballot_sync(FULL, empty);
         while (mask) {
            const int bit = __ffs(mask) - 1;
            mask &= mask - 1;
            T *zr = p.z + (base + bit) * p.ldz;
            for (long long t = lane; t < p.k; t += 32) zr[t] = T(0);
         }
      }
   }
}

template <typename T, int VOPC, int ROPC, int VSCC, int AOPC, int G, int NV>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
fused_stream_kernel(const Params<T> p)
{
   constexpr int W = VecOf<T>::W;
   constexpr int S = 32 / G;
   extern __shared__ __align__(16) unsigned char fmm_smem[];
   // ring of this warp: `depth` stages x NV vectors x 512 bytes (16 bytes per lane): for a given stage
   // and vector the 32 lanes' slots are contiguous, so the shared-memory accesses are conflict-free
   constexpr int B = G < 8 ? G : 8;                         // edges per segment
   const unsigned depth = static_cast<unsigned>(p.depth);  // power of two, B <= depth <= 32
   const unsigned ring = static_cast<unsigned>(__cvta_generic_to_shared(fmm_smem)) +
                         (threadIdx.x >> 5) * depth * NV * 512u + (threadIdx.x & 31) * 16u;
   const int vop = pick<VOPC>(p.vop), rop = pick<ROPC>(p.rop), vsc = pick<VSCC>(p.vsc), aop = pick<AOPC>(p.aop);
   const int lane = threadIdx.x & 31, lg = lane % G, slot = lane / G;
   const unsigned vmask = (G == 32) ? FULL : (((1u << G) - 1u) << (slot * G));
   (void)vmask;
   const bool need_x = vop_reads_x(vop) || rop_reads_x(rop);
   const bool need_y = vop_reads_y(vop);
   const bool use_val = (rop == ROP_NOOP) && (vsc != VSC_NOOP);
   const bool use_sop_udef = (p.sop == OP_UDEF);

   const StreamShape sh = stream_shape(p);
   if (sh.nq > p.part_cap) return;  // scratch too small: nothing is written, the host enlarges it and reruns
   const int wpc = blockDim.x >> 5;
   const long long stride = static_cast<long long>(gridDim.x) * wpc * S;

   bool inb[NV];
   long long eoff[NV];
#pragma unroll
   for (int v = 0; v < NV; v++) {
      eoff[v] = static_cast<long long>(v * G + lg) * W;
      inb[v] = eoff[v] < p.k;
   }

   for (long long w = (static_cast<long long>(blockIdx.x) * wpc + (threadIdx.x >> 5)) * S + slot;; w += stride) {
      const bool active = w < sh.nq;
      if (!__any_sync(FULL, active)) return;
      const long long a = sh.e0 + w * p.quantum;
      long long b = a + p.quantum < sh.e1 ? a + p.quantum : sh.e1;
      if (!active) b = a;  // an idle virtual warp walks an empty range in lockstep with its neighbours

      // ---- state of the row walk ---------------------------------------------------------------
      long long r = p.m, row_start = POS_INF_LL, re0 = POS_INF_LL, re1 = POS_INF_LL;
      T acc[NV][W], xv[NV][W], xn[NV][W];
#pragma unroll
      for (int v = 0; v < NV; v++)
#pragma unroll
         for (int i = 0; i < W; i++) { acc[v][i] = aop_identity<T>(aop); xv[v][i] = T(0); xn[v][i] = T(0); }
      if (active) {
         r = (w == 0) ? 0 : __ldg(p.part + w);
         if (r < p.m) {
            row_start = ld_index(p.pntrb, r, p.ptr64);
            re0 = ld_index(p.pntre, r, p.ptr64);
            if (r + 1 < p.m) re1 = ld_index(p.pntre, r + 1, p.ptr64);
            if (need_x) {
#pragma unroll
               for (int v = 0; v < NV; v++) {
                  if (inb[v]) ld_vec(p.x + r * p.ldx + eoff[v], xv[v]);
                  if (inb[v] && r + 1 < p.m) ld_vec(p.x + (r + 1) * p.ldx + eoff[v], xn[v]);
               }
            }
         }
      }
      // Stores the finished (or, for the row that began before this quantum, partial) row r and
      // moves to row r+1.  Runs with the whole virtual warp, possibly diverged from its neighbours;
      // contains no shuffles.
      auto flush_advance = [&]() {
         if (re0 > row_start) {  // rows without edges were zero-filled by the partition pass
            const bool to_z = row_start >= a;
            T *dst = to_z ? p.z + r * p.ldz : p.heads + w * p.k;
#pragma unroll
            for (int v = 0; v < NV; v++) {
               if (inb[v]) {
                  if (to_z && p.accumulate) {
                     T old[W];
                     ld_vec(dst + eoff[v], old);
#pragma unroll
                     for (int i = 0; i < W; i++) acc[v][i] = aop_apply(aop, old[i], acc[v][i]);
                  }
                  st_vec(dst + eoff[v], acc[v]);
               }
            }
         }
         row_start = re0;
         r += 1;
         re0 = (r < p.m) ? re1 : POS_INF_LL;
         re1 = (r + 1 < p.m) ? ld_index(p.pntre, r + 1, p.ptr64) : POS_INF_LL;
#pragma unroll
         for (int v = 0; v < NV; v++) {
#pragma unroll
            for (int i = 0; i < W; i++) { acc[v][i] = aop_identity<T>(aop); xv[v][i] = xn[v][i]; xn[v][i] = T(0); }
            if (need_x && inb[v] && r + 1 < p.m) ld_vec(p.x + (r + 1) * p.ldx + eoff[v], xn[v]);
         }
      };

      // ---- the edge walk -------------------------------------------------------------------------
      // Neighbour rows travel global -> shared memory with cp.async (16 bytes per lane and vector,
      // L2 only), `depth` edges ahead of the one being consumed.  Every lane copies exactly the bytes
      // it later reads back, so completion is tracked per thread with cp.async groups: no barrier, no
      // spin-wait, and the gathers in flight cost shared memory instead of registers.
      //
      // Edges are consumed in segments of up to B edges of one row, in two passes over the staged
      // rows.  Pass 1 leaves every lane with its share of each edge's reduction; one transposing
      // shuffle reduction (B-1 + log2(G/B) shuffles for B edges instead of B*log2(G)) hands the total
      // of edge e to lanes e*G/B.., where SOP runs once for all B edges; pass 2 fetches each edge's
      // scalar with one shuffle and accumulates.  The B edges of a pass are independent, which is what
      // keeps the pipelines busy with the few warps the register budget allows.
      const long long count = b - a;
      T yv[NV][W];
#pragma unroll
      for (int v = 0; v < NV; v++)
#pragma unroll
         for (int q = 0; q < W; q++) yv[v][q] = T(0);  // vectors past K are never copied and stay 0

      auto issue_gather = [&](long long j) {  // edge j of this quantum into its ring stage; one group per edge
         if (j < count && need_y) {
            const long long cid = ld_index(p.indx, a + j, p.idx64);  // same address for the G lanes: one broadcast load
            const T *yrow = p.y + cid * p.ldy;
            const unsigned st = static_cast<unsigned>(j) & (depth - 1);
#pragma unroll
            for (int v = 0; v < NV; v++)
               if (inb[v]) cp_async_16(ring + (st * NV + v) * 512u, yrow + eoff[v]);
         }
         cp_async_commit();
      };
      for (unsigned d = 0; d < depth; d++) issue_gather(d);

      long long i = 0;
      while (__any_sync(FULL, i < count)) {
         int len = 0;
         if (i < count) {
            while (a + i >= re0) flush_advance();  // leave finished (and empty) rows behind
            const long long in_row = re0 - (a + i), left = count - i;
            len = static_cast<int>(in_row < left ? in_row : left);
            len = len < B ? len : B;
         }
         cp_async_wait_pending(depth - B);  // the groups of edges i .. i+B-1 have landed
         // ---- pass 1: per-lane shares of the reductions ------------------------------------------
         T part[B];
#pragma unroll
         for (int e = 0; e < B; e++) part[e] = T(0);
         if (rop != ROP_NOOP) {
#pragma unroll
            for (int e = 0; e < B; e++) {
               if (e < len) {
                  const unsigned st = static_cast<unsigned>(i + e) & (depth - 1);
#pragma unroll
                  for (int v = 0; v < NV; v++)
                     if (need_y && inb[v]) ld_shared_vec(ring + (st * NV + v) * 512u, yv[v]);
                  T ps = T(0);
#pragma unroll
                  for (int v = 0; v < NV; v++)
#pragma unroll
                     for (int q = 0; q < W; q++) ps += rop_term(rop, xv[v][q], vop_apply(vop, xv[v][q], yv[v][q]));
                  part[e] = ps;
               }
            }
            // transposing reduction: after step k a lane keeps B >> (k+1) values
#pragma unroll
            for (int half = B / 2, off = G / 2; half >= 1; half >>= 1, off >>= 1) {
               const bool upper = (lg & off) != 0;
#pragma unroll
               for (int t = 0; t < half; t++) {
                  const T keep = upper ? part[t + half] : part[t];
                  const T send = upper ? part[t] : part[t + half];
                  part[t] = keep + __shfl_xor_sync(FULL, send, off);
               }
            }
#pragma unroll
            for (int off = G / (2 * B); off > 0; off >>= 1) part[0] += __shfl_xor_sync(FULL, part[0], off);
         } else if (use_val) {
            const int e_mine = lg / (G / B);  // this lane evaluates SOP for edge e_mine of the segment
            if (e_mine < len) part[0] = __ldg(p.val + a + i + e_mine);
         }
         const T out_mine = use_sop_udef ? sop_udef(part[0], p.sop_kind, p.sp0, p.sp1, p.sp2, p.sop_table) : part[0];
         // ---- pass 2: scale and accumulate ----------------------------------------------------------
#pragma unroll
         for (int e = 0; e < B; e++) {
            if (!__any_sync(FULL, e < len)) break;
            const T out = __shfl_sync(FULL, out_mine, e * (G / B), G);
            if (e < len) {
               const unsigned st = static_cast<unsigned>(i + e) & (depth - 1);
#pragma unroll
               for (int v = 0; v < NV; v++)
                  if (need_y && inb[v]) ld_shared_vec(ring + (st * NV + v) * 512u, yv[v]);
#pragma unroll
               for (int v = 0; v < NV; v++)
#pragma unroll
                  for (int q = 0; q < W; q++) {
                     T tt = vop_apply(vop, xv[v][q], yv[v][q]);
                     if (vsc == VSC_MUL) tt = out * tt;
                     else if (vsc == VSC_ADD) tt = out + tt;
                     acc[v][q] = aop_apply(aop, acc[v][q], tt);
                  }
            }
         }
         // ---- the stages of the segment are free again (their values were consumed above): refill ---
#pragma unroll
         for (int e = 0; e < B; e++)
            if (e < len) issue_gather(i + depth + e);
         i += len;
      }
      cp_async_wait_pending(0);
      const long long pos = a + count;
      (void)pos;
      // ---- rows that end inside (a, b], then the row that continues past b -----------------------
      if (active) {
         while (r < p.m && re0 <= b) flush_advance();
         if (r < p.m && row_start < b) {  // re0 > b: the row goes on in the next quantum
            const bool to_z = row_start >= a;
            T *dst = to_z ? p.z + r * p.ldz : p.heads + w * p.k;
#pragma unroll
            for (int v = 0; v < NV; v++) {
               if (inb[v]) {
                  if (to_z && p.accumulate) {
                     T old[W];
                     ld_vec(dst + eoff[v], old);
#pragma unroll
                     for (int i = 0; i < W; i++) acc[v][i] = aop_apply(aop, old[i], acc[v][i]);
                  }
                  st_vec(dst + eoff[v], acc[v]);
               }
            }
         }
      }
   }
}

// Pass 3: a row that crosses quantum boundaries has its first piece in Z and one head per further
// quantum.  The warp of the first boundary inside the row adds the heads to Z[row] in quantum order.
template <typename T>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32) stream_fixup_kernel(const Params<T> p)
{
   const StreamShape sh = stream_shape(p);
   if (sh.nq > p.part_cap) return;
   const int lane = threadIdx.x & 31;
   const int wpc = blockDim.x >> 5;
   const long long stride = static_cast<long long>(gridDim.x) * wpc;
   for (long long w = 1 + static_cast<long long>(blockIdx.x) * wpc + (threadIdx.x >> 5); w < sh.nq; w += stride) {
      const long long a = sh.e0 + w * p.quantum;
      const long long r = __ldg(p.part + w);  // row that holds edge a
      if (r >= p.m) continue;
      const long long rs = ld_index(p.pntrb, r, p.ptr64), re = ld_index(p.pntre, r, p.ptr64);
      if (!(rs < a && a < re)) continue;       // boundary w does not cut a row
      if (rs < a - p.quantum) continue;        // an earlier boundary also cuts this row: its warp does the sum
      T *zr = p.z + r * p.ldz;
      for (long long t = lane; t < p.k; t += 32) {
         T v = zr[t];
         for (long long q = w; q < sh.nq && sh.e0 + q * p.quantum < re; q++) v = aop_apply(p.aop, v, p.heads[q * p.k + t]);
         zr[t] = v;
      }
   }
}

}  // namespace fmm
