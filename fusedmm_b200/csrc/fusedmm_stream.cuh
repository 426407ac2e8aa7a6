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

template <typename T, int VOPC, int ROPC, int VSCC, int AOPC, int G, int NV, int U>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
fused_stream_kernel(const Params<T> p)
{
   constexpr int W = VecOf<T>::W;
   constexpr int S = 32 / G;
   static_assert(G % U == 0, "U must divide G");
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
      // Gather buffers.  Zeroed once: vectors past the end of the row (K < G*NV*W) are never loaded and
      // must stay 0 for the reductions; a skipped gather (edge slot past the end of the quantum) leaves
      // an older row behind, which is harmless because its result is not accumulated.
      T yv[U][NV][W];
#pragma unroll
      for (int u = 0; u < U; u++)
#pragma unroll
         for (int v = 0; v < NV; v++)
#pragma unroll
            for (int i = 0; i < W; i++) yv[u][v][i] = T(0);
      long long pos = a;
      while (__any_sync(FULL, pos < b)) {
         const int nb = pos < b ? ((b - pos) < G ? static_cast<int>(b - pos) : G) : 0;
         const long long j = pos + lg;
         const long long my_cid = (lg < nb && need_y) ? ld_index(p.indx, j, p.idx64) : 0;
         const T my_val = (use_val && lg < nb) ? __ldg(p.val + j) : T(0);
#pragma unroll 1
         for (int t = 0; t < G; t += U) {
            if (!__any_sync(FULL, t < nb)) break;
#pragma unroll
            for (int u = 0; u < U; u++) {
               const int e = t + u;
               const bool ok = e < nb;
               const long long cid = p.idx64 ? (static_cast<long long>(__shfl_sync(FULL, static_cast<int>(my_cid >> 32), e, G)) << 32) |
                                                  static_cast<unsigned int>(__shfl_sync(FULL, static_cast<int>(my_cid), e, G))
                                             : static_cast<long long>(__shfl_sync(FULL, static_cast<int>(my_cid), e, G));
               const T *yrow = p.y + cid * p.ldy;
#pragma unroll
               for (int v = 0; v < NV; v++)
                  if (need_y && ok && inb[v]) ld_vec_nc(yrow + eoff[v], yv[u][v]);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
               const int e = t + u;
               const bool ok = e < nb;
               if (ok) {
                  const long long eg = pos + e;
                  while (eg >= re0) flush_advance();
               }
               T tv[NV][W];
               T s = T(0);
#pragma unroll
               for (int v = 0; v < NV; v++)
#pragma unroll
                  for (int i = 0; i < W; i++) {
                     tv[v][i] = vop_apply(vop, xv[v][i], yv[u][v][i]);
                     if (rop != ROP_NOOP) s += rop_term(rop, xv[v][i], tv[v][i]);
                  }
               if (rop != ROP_NOOP) {
#pragma unroll
                  for (int off = G / 2; off > 0; off >>= 1) s += __shfl_xor_sync(FULL, s, off);
               } else {
                  s = __shfl_sync(FULL, my_val, e, G);
               }
               const T out = use_sop_udef ? sop_udef(s, p.sop_kind, p.sp0, p.sp1, p.sp2, p.sop_table) : s;
               if (ok) {
#pragma unroll
                  for (int v = 0; v < NV; v++)
#pragma unroll
                     for (int i = 0; i < W; i++) {
                        T tt = tv[v][i];
                        if (vsc == VSC_MUL) tt = out * tt;
                        else if (vsc == VSC_ADD) tt = out + tt;
                        acc[v][i] = aop_apply(aop, acc[v][i], tt);
                     }
               }
            }
         }
         pos += nb;
      }
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
