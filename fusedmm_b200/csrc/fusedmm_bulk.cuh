// fusedmm_bulk.cuh -- the chunk launch with neighbour rows staged through shared memory by bulk copies.
//
// Same work as fused_vec_kernel in MODE_HUB_CHUNKS (one warp per chunk of a split row, partial sum to
// partials[chunk]; HipGraph/FusedMM fusedMM.c:698-739 for the arithmetic), other data path: instead of every lane
// loading its 16-byte pieces of Y_v into registers, ONE lane per neighbour row issues a bulk asynchronous copy
// (cp.async.bulk, the copy engine the tensor-map TMA instructions also use; here untiled: one contiguous row) of the
// whole row from this GPU's memory into a per-warp ring in shared memory, completed by an mbarrier.  The lanes then
// read their pieces from shared memory.  What that changes:
//   * the gathered rows no longer live in registers (U x NV x 16 bytes per lane in fused_vec_kernel), so the kernel
//     fits a smaller register budget and more warps are resident;
//   * D rows per warp are in flight whatever the register budget, and a slot is refilled as soon as it is consumed;
//   * column ids need no broadcast: lane i issues the copy of "its" edge of the batch;
//   * address arithmetic runs on the issuing lane only.
// A ring slot is written by the copy engine (async proxy) and read by the lanes (generic proxy); the order is
// kept by the slot's mbarrier (copy -> read) and by __syncwarp + fence.proxy.async before a slot is reused
// (read -> next copy).  Every wait is bounded: after BULK_SPIN_LIMIT polls the warp records an error, drains what it
// has in flight (bounded again) and leaves; the host turns the error word into a status.
// The copies are plain (no cluster multicast form of any kind); source rows are in this GPU's own memory.
#pragma once
#include "fusedmm_kernels.cuh"

namespace fmm {

constexpr int BULK_SPIN_LIMIT = 1 << 22;

__device__ __forceinline__ unsigned smem_u32(const void *p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count)
{
   asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes)
{
   asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar)
{
   asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity)
{
   unsigned ok;
   asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
   return ok != 0;
}
// one contiguous row: global -> this CTA's shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_copy_row(unsigned dst, const void *src, unsigned bytes, unsigned bar)
{
   asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ void lds_vec(unsigned addr, T (&out)[VecOf<T>::W]);
template <>
__device__ __forceinline__ void lds_vec<float>(unsigned addr, float (&out)[4])
{
   asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3]) : "r"(addr) : "memory");
}
template <>
__device__ __forceinline__ void lds_vec<double>(unsigned addr, double (&out)[2])
{
   asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];" : "=d"(out[0]), "=d"(out[1]) : "r"(addr) : "memory");
}

// D = ring slots per warp (rows in flight), a power of two <= 32; U = edges per slot whose reductions are transposed
// together (as in VecEngine); S*U must divide D.
template <typename T, int VOPC, int ROPC, int VSCC, int AOPC, int G, int NV, int U, int D, int MB>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32, MB)
fused_bulk_chunk_kernel(const Params<T> p)
{
   constexpr int W = VecOf<T>::W;
   constexpr int S = 32 / G;
   constexpr int ROWB = G * NV * 16;  // bytes of a ring slot
   static_assert(D <= 32 && (D & (D - 1)) == 0 && D % (S * U) == 0, "ring size");
   static_assert(U <= G && (U & (U - 1)) == 0, "U must be a power of two no larger than G");
   extern __shared__ __align__(128) unsigned char bulk_smem[];
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
   const int wpc = blockDim.x >> 5;
   const int vop = pick<VOPC>(p.vop), rop = pick<ROPC>(p.rop), vsc = pick<VSCC>(p.vsc), aop = pick<AOPC>(p.aop);
   const int lg = lane % G, slot = lane / G;
   const bool need_x = vop_reads_x(vop) || rop_reads_x(rop);
   const bool use_val = (rop == ROP_NOOP) && (vsc != VSC_NOOP);
   const bool use_sop_udef = (p.sop == OP_UDEF);
   const int u_mine = lg / (G / U);

   unsigned char *ring = bulk_smem + static_cast<size_t>(warp) * D * ROWB;
   const unsigned ring_u32 = smem_u32(ring);
   const unsigned bars_u32 = smem_u32(bulk_smem + static_cast<size_t>(wpc) * D * ROWB) + warp * D * 8;
   if (lane < D) mbar_init(bars_u32 + lane * 8, 1);
   asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
   __syncwarp();

   grid_dependency_wait();  // the split-row list comes from the scan that precedes this launch
   const unsigned long long c = *p.counter;
   const long long nh = static_cast<long long>(c >> HUB_SHIFT);
   const long long nchunks = static_cast<long long>(c & HUB_CHUNK_MASK);
   if (nh > p.hub_cap || nchunks > p.chunk_cap) return;
   const unsigned row_bytes = static_cast<unsigned>(p.k * sizeof(T));
   unsigned batch_no = 0;  // every slot's barrier completes one phase per batch, so its parity is batch_no & 1
   bool failed = false;

   long long wid = static_cast<long long>(blockIdx.x) * wpc + warp;
   const long long stride = static_cast<long long>(gridDim.x) * wpc;
   for (; wid < nchunks && !failed; wid += stride) {
      WorkItem w;
      chunk_item(p, wid, nh, w);
      const long long n = w.ee - w.eb;

      bool inb[NV];
      T xv[NV][W], acc[NV][W];
#pragma unroll
      for (int v = 0; v < NV; v++) {
         const long long e0 = static_cast<long long>(v * G + lg) * W;
         inb[v] = e0 < p.k;
#pragma unroll
         for (int i = 0; i < W; i++) { xv[v][i] = T(0); acc[v][i] = aop_identity<T>(aop); }
         if (need_x && inb[v]) ld_vec(p.x + w.row * p.ldx + e0, xv[v]);
      }

      // lane i of a batch owns edge base + i: it loads that edge's column id and issues the copy into slot i
      auto issue = [&](long long e, long long cid) {
         const unsigned bar = bars_u32 + lane * 8;
         fence_async_proxy();  // the lanes' reads of this slot (generic proxy) come before the copy engine's write
         if (e < n) {
            mbar_expect_tx(bar, row_bytes);
            bulk_copy_row(ring_u32 + lane * ROWB, p.y + cid * p.ldy, row_bytes, bar);
         } else {
            mbar_arrive(bar);  // an unused slot still completes its phase, so all slots share one parity
         }
      };
      long long my_cid = (lane < D && lane < n) ? ld_index(p.indx, w.eb + lane, p.idx64) : 0;
      if (lane < D) issue(lane, my_cid);

      for (long long base = 0; base < n && !failed; base += D, batch_no++) {
         const int cnt = n - base < D ? static_cast<int>(n - base) : D;
         const unsigned parity = batch_no & 1;
         // next batch: column id and edge value of "my" edge, fetched a whole batch ahead of their use
         const long long nxt = base + D + lane;
         const long long next_cid = (lane < D && nxt < n) ? ld_index(p.indx, w.eb + nxt, p.idx64) : 0;
         const T my_val = (use_val && lane < D && base + lane < n) ? __ldg(p.val + w.eb + base + lane) : T(0);
#pragma unroll 1
         for (int t = 0; t < cnt; t += S * U) {
            T part[U];
            bool ok[U];
            // ---- pass 1: wait for the U rows of this slot, form the lane's share of each reduction ------
#pragma unroll
            for (int u = 0; u < U; u++) {
               const int e = t + u * S + slot;
               ok[u] = e < cnt;
               T ps[W];
#pragma unroll
               for (int i = 0; i < W; i++) ps[i] = T(0);
               if (e < D) {  // slots of this batch that carry no edge have completed their phase by a plain arrive
                  int spins = 0;
                  while (!mbar_try_wait(bars_u32 + e * 8, parity)) {
                     if (++spins > BULK_SPIN_LIMIT) { failed = true; break; }
                  }
               }
               if (ok[u] && rop != ROP_NOOP) {
#pragma unroll
                  for (int v = 0; v < NV; v++) {
                     T yv[W];
#pragma unroll
                     for (int i = 0; i < W; i++) yv[i] = T(0);
                     if (inb[v]) lds_vec<T>(ring_u32 + e * ROWB + (v * G + lg) * 16, yv);
#pragma unroll
                     for (int i = 0; i < W; i++) {
                        const T tt = vop_apply(vop, xv[v][i], yv[i]);
                        ps[i] += rop_term(rop, xv[v][i], tt);
                     }
                  }
               }
               part[u] = ps[0];
#pragma unroll
               for (int i = 1; i < W; i++) part[u] += ps[i];
            }
            if (__any_sync(FULL, failed)) { failed = true; break; }
            if (rop != ROP_NOOP) {
#pragma unroll
               for (int half = U / 2, off = G / 2; half >= 1; half >>= 1, off >>= 1) {
                  const bool upper = (lg & off) != 0;
#pragma unroll
                  for (int q = 0; q < half; q++) {
                     const T keep = upper ? part[q + half] : part[q];
                     const T send = upper ? part[q] : part[q + half];
                     part[q] = keep + __shfl_xor_sync(FULL, send, off);
                  }
               }
#pragma unroll
               for (int off = G / (2 * U); off > 0; off >>= 1) part[0] += __shfl_xor_sync(FULL, part[0], off);
            } else {
               part[0] = __shfl_sync(FULL, my_val, (t + u_mine * S + slot) & 31);  // a_uv of "my" edge
            }
            const T out_mine = use_sop_udef ? sop_udef(part[0], p.sop_kind, p.sp0, p.sp1, p.sp2, p.sop_table) : part[0];
            // ---- pass 2: the rows once more from shared memory, scaled and accumulated ------------------
#pragma unroll
            for (int u = 0; u < U; u++) {
               const T out = __shfl_sync(FULL, out_mine, u * (G / U), G);
               const int e = t + u * S + slot;
               if (ok[u]) {
#pragma unroll
                  for (int v = 0; v < NV; v++) {
                     T yv[W];
#pragma unroll
                     for (int i = 0; i < W; i++) yv[i] = T(0);
                     if (inb[v]) lds_vec<T>(ring_u32 + e * ROWB + (v * G + lg) * 16, yv);
#pragma unroll
                     for (int i = 0; i < W; i++) {
                        T tt = vop_apply(vop, xv[v][i], yv[i]);
                        if (vsc == VSC_MUL) tt = out * tt;
                        else if (vsc == VSC_ADD) tt = out + tt;
                        acc[v][i] = aop_apply(aop, acc[v][i], tt);
                     }
                  }
               }
            }
            // ---- the S*U slots t .. t+S*U-1 are consumed: their owners refill them for the next batch ----
            __syncwarp();
            if (lane >= t && lane < t + S * U && base + D < n) issue(nxt, next_cid);
         }
      }
      if (failed) break;
      // combine the edge slots and store the partial sum of the chunk
#pragma unroll
      for (int off = G; off < 32; off <<= 1)
#pragma unroll
         for (int v = 0; v < NV; v++)
#pragma unroll
            for (int i = 0; i < W; i++) acc[v][i] = aop_apply(aop, acc[v][i], __shfl_xor_sync(FULL, acc[v][i], off));
      if (lane < G) {
         T *dst = p.partials + w.dst_item * p.k;
#pragma unroll
         for (int v = 0; v < NV; v++) {
            const long long e0 = static_cast<long long>(v * G + lane) * W;
            if (e0 < p.k) st_vec(dst + e0, acc[v]);
         }
      }
   }
   if (failed) {
      // a wait ran out: record it, then give every copy this warp may still have in flight a bounded time to land
      if (lane == 0) atomicExch(p.error, 1ull);
      if (lane < D) {
         int spins = 0;
         while (!mbar_try_wait(bars_u32 + lane * 8, batch_no & 1) && ++spins < BULK_SPIN_LIMIT) {}
      }
   }
}

}  // namespace fmm
