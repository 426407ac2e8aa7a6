// fusedmm_kernels.cuh -- device code of libfusedmm_b200 (sm_100a).
//
// The operation (HipGraph/FusedMM fusedMM.c:698-739): for every row u and every edge (u,v)
//     T   = VOP(X_u, Y_v)          K-vector
//     s   = ROP(X_u, T)  or a_uv   scalar
//     out = SOP(s)                 scalar
//     T   = VSC(out, T)            K-vector
//     Z_u = AOP(Z_u, T)            K-vector
// It is a gather-bound sparse contraction (about one flop per gathered byte), so the design goal is
// bytes in flight, not tensor-core math:
//   * one warp owns one row (or one fixed-size chunk of a long row) and keeps X_u and the Z_u
//     accumulator in registers for the whole row;
//   * the warp is cut into 32/G "edge slots" of G lanes; a slot gathers one neighbour row Y_v with
//     NV 16-byte loads per lane (lane l of the slot reads vectors l, l+G, l+2G, ... so every load
//     instruction covers one contiguous G*16-byte piece of the row), and U such gathers per slot are
//     issued before the first one is consumed;
//   * the 32 column ids of a batch are fetched with one coalesced load and handed out by shuffle;
//   * ROP is a log2(G)-step shuffle reduction inside the slot, SOP/VSC/AOP run in registers, and no
//     per-edge score is ever written to memory;
//   * rows longer than `chunk` edges are cut into chunks that other warps process; their partial
//     sums go to a scratch buffer and a small second kernel adds them in chunk order, so the result
//     does not depend on scheduling (no floating-point atomics).
// This file is also the source the library hands to NVRTC at run time to build message-specific kernels
// (fusedmm_jit.cu), so it includes nothing else when compiled that way.
#pragma once
#ifndef __CUDACC_RTC__
#include <cuda_runtime.h>
#include <stdint.h>
#else
typedef unsigned long long uintptr_t;
#endif

namespace fmm {

// stage codes = the nibbles of `imessage` (reference fusedMM.h:18-73)
enum : int { VOP_NOOP = 0, VOP_COPY_LHS = 1, VOP_COPY_RHS = 2, VOP_ADD = 3, VOP_SUBL = 4, VOP_SUBR = 5,
             VOP_MAX = 6, VOP_MIN = 7, OP_UDEF = 15 };
enum : int { ROP_NOOP = 0, ROP_DOT = 1, ROP_ADD_LHS = 2, ROP_ADD_RHS = 3, ROP_NORML = 4, ROP_NORMR = 5 };
enum : int { SOP_NOOP = 0, SOP_COPY = 1 };
enum : int { VSC_NOOP = 0, VSC_MUL = 1, VSC_ADD = 2 };
enum : int { AOP_NOOP = 0, AOP_ADD = 1, AOP_MAX = 2, AOP_MIN = 3 };
enum : int { RT = -1 };  // "decided at run time": template value for the flag-interpreting kernel

// scalar functions that SOP_UDEF can stand for (include/fusedmm_b200.h FUSEDMM_SOP_*)
enum : int { SOPK_IDENTITY = 0, SOPK_SIGMOID = 1, SOPK_SIGMOID_TABLE_C = 2, SOPK_FR = 3, SOPK_TDIST = 4,
             SOPK_TDIST_CLAMPED = 5, SOPK_LL = 6, SOPK_FA = 7, SOPK_AFFINE_RECIP = 8 };

enum : int { MODE_ROWS = 0, MODE_HUB_CHUNKS = 1 };

constexpr unsigned FULL = 0xffffffffu;
// packed counter: split rows in the high 28 bits, chunks in the low 36.  2^28 split rows need more than 2^36
// edges at the smallest chunk length, beyond what one GPU's memory holds, so neither field can carry.
constexpr int HUB_SHIFT = 36;
constexpr unsigned long long HUB_CHUNK_MASK = (1ull << HUB_SHIFT) - 1ull;
constexpr int SM_TABLE_SIZE = 2048;

template <typename T>
struct Params {
   // CSR, four-array form (fusedMM.h:84-87); entry widths are run-time properties
   const void *pntrb, *pntre, *indx;
   const T *val;
   const T *x, *y;
   T *z;
   long long m, k, ldx, ldy, ldz;
   int ptr64, idx64;
   int vop, rop, sop, vsc, aop;  // stage codes of this call
   int sop_kind;                 // SOPK_* used when sop == OP_UDEF
   T sp0, sp1, sp2;              // parameters of SOPK_AFFINE_RECIP
   const T *sop_table;           // 2048-entry sigmoid table (SOPK_SIGMOID_TABLE_C)
   int accumulate;               // 1: Z = AOP(Z, result)   0: Z = result
   int mode;                     // MODE_ROWS | MODE_HUB_CHUNKS
   long long chunk;              // rows with more edges than this are split
   // hub-row scratch (written by scan_hub_rows, read by the chunk and fix-up passes)
   unsigned long long *counter;  // packed (hub rows << HUB_SHIFT) | chunks
   long long *hub_row, *hub_base;
   long long hub_cap, chunk_cap;
   T *partials;                  // chunk_cap x k
   // optional visiting order of the chunks (order[i] = chunk the i-th work item works on; null: i itself): chunks
   // sorted by the column id of their first edge, so that the chunks in flight at one time gather from one band of Y
   const long long *order;
   // optional order of the whole rows (row_order[i] = row of the i-th slot of the whole-row launch; null: i itself):
   // rows sorted by their number of edges inside windows of consecutive rows, so that the rows that share a warp
   // (32/G of them, in lockstep) are about equally long
   const unsigned int *row_order;
   // edge-stream scheduler (fusedmm_stream.cuh): the edges are cut into quanta of `quantum` edges
   long long quantum;            // edges per work item (a multiple of 32)
   int depth;                    // neighbour rows in flight per virtual warp (power of two <= lanes per edge)
   long long *part;              // part[w] = row that holds the first edge of quantum w   (part_cap+1 entries)
   long long part_cap;           // quanta the scratch has room for
   T *heads;                     // heads[w] = partial sum of the row that straddles the start of quantum w
   // optional replication of the finished Z rows into other GPUs' Z buffers (multi-GPU all-gather
   // fused into the epilogue); z_peer[i] has the same layout as z
   int n_peers;
   T *z_peer[8];
   // or: one multicast address of Z (an NVSwitch multicast object that maps the same buffer on every
   // GPU of the group, this GPU included): a finished row is then stored ONCE with multimem.st and the
   // switch delivers it to every GPU, so a rank sends its shard once instead of once per peer
   T *z_mc;
   // 1: rows without edges are not sent to the other GPUs (every GPU holds the row pointers and zeroes, or
   // keeps, those rows of its own copy itself: zero_empty_rows_kernel); their result is stored locally only
   int skip_empty_remote;
   unsigned long long *error;    // set to 1 by a kernel whose bounded wait ran out (fusedmm_bulk.cuh); read by the host
   // host side only: launch this kernel with programmatic stream serialization (it may become resident while the
   // kernel before it in the stream is still running and waits at grid_dependency_wait for that kernel's results)
   int pdl;
};

// ---------------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------------
template <int C>
__device__ __forceinline__ int pick(int rt) { return C >= 0 ? C : rt; }

__device__ __forceinline__ long long ld_index(const void *a, long long j, int is64)
{
   return is64 ? __ldg(reinterpret_cast<const long long *>(a) + j)
               : static_cast<long long>(__ldg(reinterpret_cast<const int *>(a) + j));
}

__device__ __forceinline__ long long shfl_ll(long long v, int src)
{
   int lo = __shfl_sync(FULL, static_cast<int>(v), src);
   int hi = __shfl_sync(FULL, static_cast<int>(v >> 32), src);
   return (static_cast<long long>(hi) << 32) | static_cast<unsigned int>(lo);
}

template <typename T> struct VecOf;
template <> struct VecOf<float>  { using type = float4;  static constexpr int W = 4; };
template <> struct VecOf<double> { using type = double2; static constexpr int W = 2; };

template <typename T>
__device__ __forceinline__ void ld_vec_nc(const T *ptr, T (&out)[VecOf<T>::W]);
template <>
__device__ __forceinline__ void ld_vec_nc<float>(const float *ptr, float (&out)[4])
{
   float4 v = __ldg(reinterpret_cast<const float4 *>(ptr));
   out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <>
__device__ __forceinline__ void ld_vec_nc<double>(const double *ptr, double (&out)[2])
{
   double2 v = __ldg(reinterpret_cast<const double2 *>(ptr));
   out[0] = v.x; out[1] = v.y;
}
template <typename T>
__device__ __forceinline__ void ld_vec(const T *ptr, T (&out)[VecOf<T>::W])
{
   using V = typename VecOf<T>::type;
   V v = *reinterpret_cast<const V *>(ptr);
   const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
   for (int i = 0; i < VecOf<T>::W; i++) out[i] = e[i];
}
template <typename T>
__device__ __forceinline__ void st_vec(T *ptr, const T (&in)[VecOf<T>::W])
{
   using V = typename VecOf<T>::type;
   V v;
   T *e = reinterpret_cast<T *>(&v);
#pragma unroll
   for (int i = 0; i < VecOf<T>::W; i++) e[i] = in[i];
   *reinterpret_cast<V *>(ptr) = v;
}

// One-element "vectors" (FLAG_ELEMENT: K, a leading dimension or a base address that is not a multiple of 16 bytes):
// the same engine with 4- or 8-byte accesses, a warp instruction still covers one contiguous G-element piece of a row.
__device__ __forceinline__ void ld_vec_nc(const float *ptr, float (&out)[1]) { out[0] = __ldg(ptr); }
__device__ __forceinline__ void ld_vec_nc(const double *ptr, double (&out)[1]) { out[0] = __ldg(ptr); }
__device__ __forceinline__ void ld_vec(const float *ptr, float (&out)[1]) { out[0] = *ptr; }
__device__ __forceinline__ void ld_vec(const double *ptr, double (&out)[1]) { out[0] = *ptr; }
__device__ __forceinline__ void st_vec(float *ptr, const float (&in)[1]) { *ptr = in[0]; }
__device__ __forceinline__ void st_vec(double *ptr, const double (&in)[1]) { *ptr = in[0]; }

// multimem.st: one store through an NVSwitch multicast address lands in every GPU's copy of the buffer
__device__ __forceinline__ void st_vec_multicast(float *mc, const float (&in)[4])
{
   asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(in[0]), "f"(in[1]),
                "f"(in[2]), "f"(in[3]) : "memory");
}
__device__ __forceinline__ void st_vec_multicast(double *mc, const double (&in)[2])
{
   // multimem.st has no .v2.f64 form; a store only moves bits, so the 16 bytes go as four 32-bit words
   asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
                "f"(__int_as_float(__double2loint(in[0]))), "f"(__int_as_float(__double2hiint(in[0]))),
                "f"(__int_as_float(__double2loint(in[1]))), "f"(__int_as_float(__double2hiint(in[1]))) : "memory");
}
__device__ __forceinline__ void st_multicast(float *mc, float v)
{
   asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}
__device__ __forceinline__ void st_multicast(double *mc, double v)
{
   asm volatile("multimem.st.relaxed.sys.global.f64 [%0], %1;" ::"l"(mc), "d"(v) : "memory");
}

// Programmatic dependent launch: a kernel launched with programmatic stream serialization must not touch what the
// kernel before it in the stream produces until this returns; without that launch attribute it is a no-op.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream (if it was launched that way) become resident now instead of when this grid
// has drained; it still waits for this grid's completion in grid_dependency_wait.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ void st_vec_multicast(float *mc, const float (&in)[1]) { st_multicast(mc, in[0]); }
__device__ __forceinline__ void st_vec_multicast(double *mc, const double (&in)[1]) { st_multicast(mc, in[0]); }

template <typename T> __device__ __forceinline__ T pos_inf();
template <> __device__ __forceinline__ float  pos_inf<float>()  { return __int_as_float(0x7f800000); }
template <> __device__ __forceinline__ double pos_inf<double>() { return __longlong_as_double(0x7ff0000000000000LL); }

// ---------------------------------------------------------------------------------------------------
// stage bodies.  lhs = X_u element, rhs = Y_v element.
// ---------------------------------------------------------------------------------------------------
// fusedMM.c:28-138.  SUBL is rhs-lhs (:87) and SUBR is lhs-rhs (:103); max/min use the reference's
// comparison macros (fusedMM.c:18-19), not IEEE fmax/fmin.
template <typename T>
__device__ __forceinline__ T vop_apply(int vop, T lhs, T rhs)
{
   switch (vop) {
      case VOP_COPY_LHS: return lhs;
      case VOP_ADD:      return lhs + rhs;
      case VOP_SUBL:     return rhs - lhs;
      case VOP_SUBR:     return lhs - rhs;
      case VOP_MAX:      return lhs > rhs ? lhs : rhs;
      case VOP_MIN:      return lhs < rhs ? lhs : rhs;
      default:           return rhs;  // VOP_COPY_RHS (and VOP_NOOP when the caller opted in)
   }
}
// per-element term of the reduction; the second operand of ROP is T (fusedMM.c:725, :144-202)
template <typename T>
__device__ __forceinline__ T rop_term(int rop, T lhs, T t)
{
   switch (rop) {
      case ROP_DOT:     return lhs * t;
      case ROP_ADD_LHS: return lhs;
      case ROP_ADD_RHS: return t;
      case ROP_NORML:   return lhs * lhs;
      default:          return t * t;  // ROP_NORMR
   }
}
__host__ __device__ __forceinline__ bool vop_reads_x(int vop) { return vop != VOP_COPY_RHS && vop != VOP_NOOP; }
__host__ __device__ __forceinline__ bool vop_reads_y(int vop) { return vop != VOP_COPY_LHS; }
__host__ __device__ __forceinline__ bool rop_reads_x(int rop) { return rop == ROP_DOT || rop == ROP_ADD_LHS || rop == ROP_NORML; }

// fusedMM.c:268-333
template <typename T>
__device__ __forceinline__ T aop_apply(int aop, T acc, T t)
{
   switch (aop) {
      case AOP_MAX: return acc > t ? acc : t;
      case AOP_MIN: return acc < t ? acc : t;
      default:      return acc + t;
   }
}
template <typename T>
__device__ __forceinline__ T aop_identity(int aop)
{
   return aop == AOP_MAX ? -pos_inf<T>() : (aop == AOP_MIN ? pos_inf<T>() : T(0));
}

// The same stage bodies over a lane's whole share of an edge, with the switch OUTSIDE the element loops: the
// flag-interpreting instantiation then pays one uniform branch per stage and edge instead of one per element.
#define FMM_FOR_VI _Pragma("unroll") for (int v = 0; v < NV; v++) _Pragma("unroll") for (int i = 0; i < W; i++)
template <typename T, int NV, int W>
__device__ __forceinline__ void vop_block(int vop, const T (&x)[NV][W], T (&y)[NV][W])
{
   switch (vop) {
      case VOP_COPY_LHS: FMM_FOR_VI y[v][i] = x[v][i]; break;
      case VOP_ADD:      FMM_FOR_VI y[v][i] = x[v][i] + y[v][i]; break;
      case VOP_SUBL:     FMM_FOR_VI y[v][i] = y[v][i] - x[v][i]; break;
      case VOP_SUBR:     FMM_FOR_VI y[v][i] = x[v][i] - y[v][i]; break;
      case VOP_MAX:      FMM_FOR_VI y[v][i] = x[v][i] > y[v][i] ? x[v][i] : y[v][i]; break;
      case VOP_MIN:      FMM_FOR_VI y[v][i] = x[v][i] < y[v][i] ? x[v][i] : y[v][i]; break;
      default: break;  // VOP_COPY_RHS: T is the gathered row
   }
}
// ps[i] += the reduction terms of this lane's elements, in the element order of rop_term's callers
template <typename T, int NV, int W>
__device__ __forceinline__ void rop_block(int rop, const T (&x)[NV][W], const T (&t)[NV][W], T (&ps)[W])
{
   switch (rop) {
      case ROP_DOT:     FMM_FOR_VI ps[i] += x[v][i] * t[v][i]; break;
      case ROP_ADD_LHS: FMM_FOR_VI ps[i] += x[v][i]; break;
      case ROP_ADD_RHS: FMM_FOR_VI ps[i] += t[v][i]; break;
      case ROP_NORML:   FMM_FOR_VI ps[i] += x[v][i] * x[v][i]; break;
      case ROP_NORMR:   FMM_FOR_VI ps[i] += t[v][i] * t[v][i]; break;
      default: break;   // ROP_NOOP
   }
}
// acc = AOP(acc, VSC(out, t))
template <typename T, int NV, int W>
__device__ __forceinline__ void vsc_aop_block(int vsc, int aop, T out, const T (&t)[NV][W], T (&acc)[NV][W])
{
   const int a = aop == AOP_MAX ? 1 : (aop == AOP_MIN ? 2 : 0);
   const int m = vsc == VSC_MUL ? 1 : (vsc == VSC_ADD ? 2 : 0);
   switch (m * 3 + a) {
      case 0: FMM_FOR_VI acc[v][i] += t[v][i]; break;
      case 1: FMM_FOR_VI { const T tt = t[v][i]; acc[v][i] = acc[v][i] > tt ? acc[v][i] : tt; } break;
      case 2: FMM_FOR_VI { const T tt = t[v][i]; acc[v][i] = acc[v][i] < tt ? acc[v][i] : tt; } break;
      case 3: FMM_FOR_VI acc[v][i] += out * t[v][i]; break;
      case 4: FMM_FOR_VI { const T tt = out * t[v][i]; acc[v][i] = acc[v][i] > tt ? acc[v][i] : tt; } break;
      case 5: FMM_FOR_VI { const T tt = out * t[v][i]; acc[v][i] = acc[v][i] < tt ? acc[v][i] : tt; } break;
      case 6: FMM_FOR_VI acc[v][i] += out + t[v][i]; break;
      case 7: FMM_FOR_VI { const T tt = out + t[v][i]; acc[v][i] = acc[v][i] > tt ? acc[v][i] : tt; } break;
      default: FMM_FOR_VI { const T tt = out + t[v][i]; acc[v][i] = acc[v][i] < tt ? acc[v][i] : tt; } break;
   }
}
#undef FMM_FOR_VI

// Scalar functions.  fp32 uses expf/logf-class functions (a few ulp), never the fast intrinsics; the
// table variant computes its index in double exactly as the host code it mirrors
// (test/fusedMMtime.cpp:606-611).
__device__ __forceinline__ float  fmm_exp(float v)  { return expf(v); }
__device__ __forceinline__ double fmm_exp(double v) { return exp(v); }
__device__ __forceinline__ float  fmm_sqrt(float v)  { return sqrtf(v); }
__device__ __forceinline__ double fmm_sqrt(double v) { return sqrt(v); }
__device__ __forceinline__ float  fmm_log2(float v)  { return log2f(v); }
__device__ __forceinline__ double fmm_log2(double v) { return log2(v); }
// log2(1 + v) without forming 1 + v: for the small v that near-equal rows give (K = 1 or 2 layouts), 1 + v in float
// keeps only a few digits of v and the logarithm inherits that error (2e-4 relative at v = 3e-4)
__device__ __forceinline__ float  fmm_log2_1p(float v)  { return log1pf(v) * 1.44269504088896340736f; }
__device__ __forceinline__ double fmm_log2_1p(double v) { return log1p(v) * 1.44269504088896340736; }

template <typename T>
__device__ __forceinline__ T sop_udef(T s, int kind, T p0, T p1, T p2, const T *table)
{
   switch (kind) {
      case SOPK_SIGMOID: return T(1) / (T(1) + fmm_exp(-s));
      case SOPK_SIGMOID_TABLE_C: {
         T sm;
         if (s > T(5)) sm = T(1);
         else if (s < T(-5)) sm = T(0);
         else {
            int idx = static_cast<int>((static_cast<double>(s) + 5.0) * SM_TABLE_SIZE / (2.0 * 5.0));
            idx = idx > SM_TABLE_SIZE - 1 ? SM_TABLE_SIZE - 1 : idx;
            sm = __ldg(table + idx);
         }
         return T(1) - sm;
      }
      case SOPK_FR:    return T(1) + T(1) / s;
      case SOPK_TDIST: return T(1) / (T(1) + s);
      case SOPK_TDIST_CLAMPED: {
         T v = T(-2) / (T(1) + s);
         return v > T(5) ? T(5) : (v < T(-5) ? T(-5) : v);
      }
      case SOPK_LL: return fmm_log2_1p(fmm_sqrt(s));
      case SOPK_FA: return fmm_sqrt(s) + T(1) / s;
      case SOPK_AFFINE_RECIP: {
         T v = p0 / (p1 + s);
         if (p2 > T(0)) v = v > p2 ? p2 : (v < -p2 ? -p2 : v);
         return v;
      }
      default: return s;
   }
}

// ---------------------------------------------------------------------------------------------------
// Work-item lookup shared by the two main kernels.
// ---------------------------------------------------------------------------------------------------
struct WorkItem {
   long long row, eb, ee;  // row and edge range [eb, ee)
   long long dst_item;     // chunk index for MODE_HUB_CHUNKS, -1 for a whole row
};

// largest slot with hub_base[slot] <= item; hub_base is increasing because slot and base come out of
// one packed atomic counter.  The whole warp searches together, 32 pivots per step: four dependent
// loads for 200 000 split rows instead of eighteen.  Every lane must call this with the same arguments.
__device__ __forceinline__ long long hub_slot_of(const long long *hub_base, long long nh, long long item)
{
   const int lane = threadIdx.x & 31;
   long long lo = 0, hi = nh;  // the answer is in [lo, hi) and hub_base[lo] <= item
   while (hi - lo > 1) {
      const long long step = (hi - lo + 31) / 32;
      const long long probe = lo + lane * step;
      const bool le = probe < hi && __ldg(hub_base + probe) <= item;
      const int cnt = __popc(__ballot_sync(FULL, le));  // the probes that are <= item form a prefix
      lo += (cnt - 1) * step;
      hi = lo + step < hi ? lo + step : hi;
   }
   return lo;
}

template <typename T>
__device__ __forceinline__ bool chunk_item(const Params<T> &p, long long item, long long nh, WorkItem &w)
{
   long long slot = hub_slot_of(p.hub_base, nh, item);
   w.row = __ldg(p.hub_row + slot);
   long long c = item - __ldg(p.hub_base + slot);
   long long pb = ld_index(p.pntrb, w.row, p.ptr64), pe = ld_index(p.pntre, w.row, p.ptr64);
   w.eb = pb + c * p.chunk;
   w.ee = w.eb + p.chunk < pe ? w.eb + p.chunk : pe;
   w.dst_item = item;
   return true;
}

// Z_row = AOP(old Z_row or identity, partial_0, partial_1, ...) in chunk order, by one warp; also sends the row to
// the other GPUs when the call asks for that.  Lane l owns elements l, l+32, ... of a 128-element tile of K; the
// loads of four chunks are in flight together while the additions keep their order.
template <typename T>
__device__ __forceinline__ void reduce_hub_row(const Params<T> &p, long long row, long long base, long long nch, int lane)
{
   constexpr int EPT = 4;
   T *zr = p.z + row * p.ldz;
   for (long long kt = 0; kt < p.k; kt += 32 * EPT) {
      T a[EPT];
#pragma unroll
      for (int e = 0; e < EPT; e++) {
         const long long t = kt + e * 32 + lane;
         a[e] = (p.accumulate && t < p.k) ? zr[t] : aop_identity<T>(p.aop);
      }
      const T *src = p.partials + base * p.k + kt + lane;
#pragma unroll 4
      for (long long q = 0; q < nch; q++, src += p.k) {
         T v[EPT];
#pragma unroll
         for (int e = 0; e < EPT; e++) v[e] = (kt + e * 32 + lane < p.k) ? __ldcg(src + e * 32) : aop_identity<T>(p.aop);
#pragma unroll
         for (int e = 0; e < EPT; e++) a[e] = aop_apply(p.aop, a[e], v[e]);
      }
#pragma unroll
      for (int e = 0; e < EPT; e++) {
         const long long t = kt + e * 32 + lane;
         if (t < p.k) {
            if (p.z_mc) {
               st_multicast(p.z_mc + row * p.ldz + t, a[e]);
            } else {
               zr[t] = a[e];
               for (int g = 0; g < p.n_peers; g++) p.z_peer[g][row * p.ldz + t] = a[e];
            }
         }
      }
   }
}

// ---------------------------------------------------------------------------------------------------
// Vector engine: one warp, one work item, K <= G*NV*W elements, everything 16-byte aligned.
// ---------------------------------------------------------------------------------------------------
// FLAGS: properties of the CALL (not of the message) that a kernel built at run time for that call may assume:
//   FLAG_EXACT_K   k == G*NV*W: no vector of the tiling lies beyond the end of a row, so the per-vector bounds
//                  predicates on every gather and store go away;
//   FLAG_OFFSET32  column ids are 32 bits wide (and not negative) and a row of Y is less than 2^32 bytes from the next:
//                  the address of a lane's piece of a neighbour row is ONE 32 x 32 + 64-bit multiply-add on the lane's
//                  own base address, instead of a 64-bit multiply, a scaled add and one 64-bit add per vector.
//   FLAG_ELEMENT   vectors of ONE element instead of 16 bytes: for calls whose K, leading dimensions or base addresses
//                  are not multiples of 16 bytes (K up to G*NV elements).
// FLAGS = 0 takes every call whose rows are 16-byte granular.
enum : int { FLAG_EXACT_K = 1, FLAG_OFFSET32 = 2, FLAG_ELEMENT = 4 };

template <typename T, int VOPC, int ROPC, int VSCC, int AOPC, int G, int NV, int U, int FLAGS = 0>
struct VecEngine {
   static constexpr int W = (FLAGS & FLAG_ELEMENT) ? 1 : VecOf<T>::W;
   static constexpr bool EXACT_K = (FLAGS & FLAG_EXACT_K) != 0;
   static constexpr bool OFFSET32 = (FLAGS & FLAG_OFFSET32) != 0;
   static constexpr int S = 32 / G;  // edge slots per warp
   // the flag-interpreting instantiation: stage codes are only known at run time
   static constexpr bool RUNTIME_CODES = VOPC < 0 || ROPC < 0 || VSCC < 0 || AOPC < 0;
   static_assert(S * U <= 32 && (32 % (S * U)) == 0, "S*U must divide 32");
   static_assert(U <= G && (U & (U - 1)) == 0, "U must be a power of two no larger than G");

   // MULTI = false: the whole warp works on ONE item; its S slots take alternate edges and their
   //                 accumulators are combined at the end (long rows and chunks of split rows).
   // MULTI = true:  every slot has its OWN item (`w` differs between slots) and walks it alone: S short
   //                 rows per warp, in lockstep, which is what keeps enough gathers in flight when the
   //                 rows have only a handful of edges.
   template <bool MULTI>
   __device__ __forceinline__ static void run(const Params<T> &p, const WorkItem &w, int lane,
                                              T (&acc)[NV][W])
   {
      constexpr int BW = MULTI ? G : 32;  // column ids fetched per batch
      constexpr int ES = MULTI ? 1 : S;   // distance between the edges u and u+1 of a slot
      const int vop = pick<VOPC>(p.vop), rop = pick<ROPC>(p.rop), vsc = pick<VSCC>(p.vsc),
                aop = pick<AOPC>(p.aop);
      const int lg = lane % G, slot = lane / G;
      const bool need_x = vop_reads_x(vop) || rop_reads_x(rop);
      const bool need_y = vop_reads_y(vop);
      const bool use_val = (rop == ROP_NOOP) && (vsc != VSC_NOOP);
      const bool use_sop_udef = (p.sop == OP_UDEF);

      bool inb[NV];
      T xv[NV][W];
#pragma unroll
      for (int v = 0; v < NV; v++) {
         const long long e0 = static_cast<long long>(v * G + lg) * W;
         inb[v] = EXACT_K || e0 < p.k;
#pragma unroll
         for (int i = 0; i < W; i++) { xv[v][i] = T(0); acc[v][i] = aop_identity<T>(aop); }
         if (need_x && inb[v] && w.eb < w.ee) ld_vec(p.x + w.row * p.ldx + e0, xv[v]);  // an item without edges reads nothing
      }

      // Gather buffers, zeroed once: vectors past the end of the row (K < G*NV*W) are never loaded
      // and must stay 0 for the reductions; a skipped gather (edge slot past the end of the row)
      // leaves older values behind, which is harmless because its result is not accumulated.
      T yv[U][NV][W];
#pragma unroll
      for (int u = 0; u < U; u++)
#pragma unroll
         for (int v = 0; v < NV; v++)
#pragma unroll
            for (int i = 0; i < W; i++) yv[u][v][i] = T(0);
      const int u_mine = lg / (G / U);  // the edge of a group whose scalar this lane ends up holding
      // FLAG_OFFSET32: byte address of this lane's first vector in row 0 of Y, and the row pitch in bytes (< 2^32)
      const char *y_lane = reinterpret_cast<const char *>(p.y + lg * W);
      const unsigned int ldy_bytes = static_cast<unsigned int>(p.ldy * static_cast<long long>(sizeof(T)));
      const int eslot = MULTI ? 0 : slot;
      const int blane = MULTI ? lg : lane;

      for (long long base = w.eb; MULTI ? __any_sync(FULL, base < w.ee) : (base < w.ee); base += BW) {
         const long long j = base + blane;
         long long my_cid = 0;
         unsigned int my_cid32 = 0;  // FLAG_OFFSET32: column ids are 32 bits wide
         if constexpr (OFFSET32) { if (j < w.ee && need_y) my_cid32 = static_cast<unsigned int>(__ldg(static_cast<const int *>(p.indx) + j)); }
         else { if (j < w.ee && need_y) my_cid = ld_index(p.indx, j, p.idx64); }
         const T my_val = (use_val && j < w.ee) ? __ldg(p.val + j) : T(0);
         const long long left = w.ee - base;
         const int nb = left < BW ? (left > 0 ? static_cast<int>(left) : 0) : BW;
#pragma unroll 1
         for (int t = 0; MULTI ? __any_sync(FULL, t < nb) : (t < nb); t += ES * U) {
            // ---- U gathers per slot in flight ------------------------------------------------------
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
               const int e = t + u * ES + eslot;  // < BW because ES*U divides BW
               ok[u] = e < nb;
               const T *yrow;
               if constexpr (OFFSET32) {
                  // one 32 x 32 + 64-bit multiply-add: the lane's byte address in the neighbour's row
                  const unsigned int cid = __shfl_sync(FULL, my_cid32, e, BW);
                  yrow = reinterpret_cast<const T *>(y_lane + static_cast<unsigned long long>(cid) * ldy_bytes);
               } else {
                  const long long cid = p.idx64 ? (static_cast<long long>(__shfl_sync(FULL, static_cast<int>(my_cid >> 32), e, BW)) << 32) |
                                                     static_cast<unsigned int>(__shfl_sync(FULL, static_cast<int>(my_cid), e, BW))
                                                : static_cast<long long>(__shfl_sync(FULL, static_cast<int>(my_cid), e, BW));
                  yrow = p.y + cid * p.ldy;
               }
#pragma unroll
               for (int v = 0; v < NV; v++)
                  if (need_y && ok[u] && inb[v]) ld_vec_nc(yrow + (OFFSET32 ? v * G * W : static_cast<long long>(v * G + lg) * W), yv[u][v]);
            }
            // ---- pass 1: T = VOP(x, y) in place, and this lane's share of each edge's reduction ----
            T part[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
               T ps[W];
#pragma unroll
               for (int i = 0; i < W; i++) ps[i] = T(0);
               if constexpr (RUNTIME_CODES) {
                  vop_block<T, NV, W>(vop, xv, yv[u]);
                  rop_block<T, NV, W>(rop, xv, yv[u], ps);
               } else {
#pragma unroll
                  for (int v = 0; v < NV; v++)
#pragma unroll
                     for (int i = 0; i < W; i++) {
                        yv[u][v][i] = vop_apply(vop, xv[v][i], yv[u][v][i]);
                        if (rop != ROP_NOOP) ps[i] += rop_term(rop, xv[v][i], yv[u][v][i]);
                     }
               }
               part[u] = ps[0];
#pragma unroll
               for (int i = 1; i < W; i++) part[u] += ps[i];
            }
            if (rop != ROP_NOOP) {
               // Transposing reduction over the G lanes of the slot: each step halves the number of
               // values a lane holds, so the U totals cost U-1 + log2(G/U) shuffles instead of
               // U*log2(G); afterwards lanes u*(G/U).. hold the total of edge u.
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
               part[0] = __shfl_sync(FULL, my_val, t + u_mine * ES + eslot, BW);  // a_uv of "my" edge
            }
            // ---- SOP once for the U edges of the group (lane group u evaluates edge u) --------------
            const T out_mine = use_sop_udef ? sop_udef(part[0], p.sop_kind, p.sp0, p.sp1, p.sp2, p.sop_table) : part[0];
            // ---- pass 2: scale and accumulate --------------------------------------------------------
#pragma unroll
            for (int u = 0; u < U; u++) {
               const T out = __shfl_sync(FULL, out_mine, u * (G / U), G);
               if (ok[u]) {
                  if constexpr (RUNTIME_CODES) {
                     vsc_aop_block<T, NV, W>(vsc, aop, out, yv[u], acc);
                  } else {
#pragma unroll
                     for (int v = 0; v < NV; v++)
#pragma unroll
                        for (int i = 0; i < W; i++) {
                           T tt = yv[u][v][i];
                           if (vsc == VSC_MUL) tt = out * tt;
                           else if (vsc == VSC_ADD) tt = out + tt;
                           acc[v][i] = aop_apply(aop, acc[v][i], tt);
                        }
                  }
               }
            }
         }
      }
      // combine the edge slots: afterwards every slot holds the row's result
#pragma unroll
      for (int off = G; !MULTI && off < 32; off <<= 1)
#pragma unroll
         for (int v = 0; v < NV; v++)
#pragma unroll
            for (int i = 0; i < W; i++)
               acc[v][i] = aop_apply(aop, acc[v][i], __shfl_xor_sync(FULL, acc[v][i], off));
   }
};

constexpr int WARPS_PER_CTA = 8;  // upper bound; the launch chooses blockDim.x = 32 * (1..8)
constexpr int ANY_MAX_CACHED = 512;  // element-strided engine: edges of an item whose scalars are kept in shared memory

// One warp per row (MODE_ROWS) or a grid-stride loop over the chunks of split rows
// (MODE_HUB_CHUNKS).  Rows longer than p.chunk are skipped in MODE_ROWS.
// MB = resident 256-thread blocks per SM the register allocation must allow (0: the compiler's choice, 2: at most
// 128 registers per thread, 3: 80, 4: 64): for some tilings a tighter budget (a few spills, more resident warps)
// is faster.
template <typename T, int VOPC, int ROPC, int VSCC, int AOPC, int G, int NV, int U, int MB, int FLAGS = 0>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32, MB)
fused_vec_kernel(const Params<T> p)
{
   using Eng = VecEngine<T, VOPC, ROPC, VSCC, AOPC, G, NV, U, FLAGS>;
   constexpr int W = Eng::W;
   constexpr bool EXACT_K = Eng::EXACT_K;
   const int lane = threadIdx.x & 31;
   const int aop = pick<AOPC>(p.aop);
   const int wpc = blockDim.x >> 5;
   long long wid = static_cast<long long>(blockIdx.x) * wpc + (threadIdx.x >> 5);
   const long long stride = static_cast<long long>(gridDim.x) * wpc;
   long long nh = 0, nchunks = 0;
   if (p.mode == MODE_HUB_CHUNKS) {
      grid_dependency_wait();  // the split-row list comes from the scan that precedes this launch
      const unsigned long long c = *p.counter;
      nh = static_cast<long long>(c >> HUB_SHIFT);
      nchunks = static_cast<long long>(c & HUB_CHUNK_MASK);
      if (nh > p.hub_cap || nchunks > p.chunk_cap) return;  // scratch too small: the host enlarges it and reruns
   }
   constexpr int S = 32 / G;
   if (S > 1 && p.mode == MODE_ROWS) {
      // short rows: every slot of the warp takes its own row
      const int lg = lane % G, slot = lane / G;
      if (wid * S >= p.m) return;
      WorkItem w;
      w.row = wid * S + slot;
      w.dst_item = -1;
      w.eb = w.ee = 0;
      bool mine = w.row < p.m;
      if (mine && p.row_order) w.row = __ldg(p.row_order + w.row);
      if (mine) {
         w.eb = ld_index(p.pntrb, w.row, p.ptr64);
         w.ee = ld_index(p.pntre, w.row, p.ptr64);
         if (w.ee - w.eb > p.chunk) { mine = false; w.ee = w.eb; }  // split rows belong to the chunk launch
      } else {
         w.row = 0;
      }
      T acc[NV][W];
      Eng::template run<true>(p, w, lane, acc);
      if (mine && p.accumulate && w.eb == w.ee) mine = false;  // accumulating nothing: the row of Z stays as it is
      if (mine) {
         T *dst = p.z + w.row * p.ldz;
#pragma unroll
         for (int v = 0; v < NV; v++) {
            const long long e0 = static_cast<long long>(v * G + lg) * W;
            if (EXACT_K || e0 < p.k) {
               if (p.accumulate) {
                  T old[W];
                  ld_vec(dst + e0, old);
#pragma unroll
                  for (int i = 0; i < W; i++) acc[v][i] = aop_apply(aop, old[i], acc[v][i]);
               }
               const bool remote = !(p.skip_empty_remote && w.eb == w.ee);
               if (p.z_mc && remote) {
                  st_vec_multicast(p.z_mc + w.row * p.ldz + e0, acc[v]);
               } else {
                  st_vec(dst + e0, acc[v]);
                  if (remote)
                     for (int q = 0; q < p.n_peers; q++) st_vec(p.z_peer[q] + w.row * p.ldz + e0, acc[v]);
               }
            }
         }
      }
      return;
   }
   for (;; wid += stride) {
      WorkItem w;
      if (p.mode == MODE_ROWS) {
         if (wid >= p.m) return;
         w.row = wid;
         w.eb = ld_index(p.pntrb, wid, p.ptr64);
         w.ee = ld_index(p.pntre, wid, p.ptr64);
         w.dst_item = -1;
         if (w.ee - w.eb > p.chunk) return;
      } else {
         if (wid >= nchunks) return;
         chunk_item(p, p.order ? __ldg(p.order + wid) : wid, nh, w);
      }
      T acc[NV][W];
      Eng::template run<false>(p, w, lane, acc);

      if (lane < G && !(w.dst_item < 0 && p.accumulate && w.eb == w.ee)) {  // slot 0 holds (like every slot) the finished sums
         const bool to_z = w.dst_item < 0;
         const bool remote = !(p.skip_empty_remote && w.eb == w.ee);
         T *dst = to_z ? p.z + w.row * p.ldz : p.partials + w.dst_item * p.k;
#pragma unroll
         for (int v = 0; v < NV; v++) {
            const long long e0 = static_cast<long long>(v * G + lane) * W;
            if (EXACT_K || e0 < p.k) {
               if (to_z && p.accumulate) {
                  T old[W];
                  ld_vec(dst + e0, old);
#pragma unroll
                  for (int i = 0; i < W; i++) acc[v][i] = aop_apply(aop, old[i], acc[v][i]);
               }
               if (to_z && p.z_mc && remote) {
                  st_vec_multicast(p.z_mc + w.row * p.ldz + e0, acc[v]);
               } else {
                  st_vec(dst + e0, acc[v]);
                  if (to_z && remote)
                     for (int q = 0; q < p.n_peers; q++) st_vec(p.z_peer[q] + w.row * p.ldz + e0, acc[v]);
               }
            }
         }
      }
      if (p.mode == MODE_ROWS) return;
   }
}

// ---------------------------------------------------------------------------------------------------
// Element-strided engine: any K, any leading dimension, any alignment; all stage codes at run time.
// Lane l owns elements l, l+32, ... of a 32*EPT-element tile of K; a message with a reduction walks
// the whole K once per edge to get s, keeps the scalars of the item's edges in shared memory and then walks
// the tiles (items of more than ANY_MAX_CACHED edges recompute s per tile).  It exists so that every legal
// call has a GPU path; the vector engine is the fast one.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
fused_any_kernel(const Params<T> p)
{
   constexpr int EPT = 8;
   const int lane = threadIdx.x & 31;
   const int vop = p.vop, rop = p.rop, vsc = p.vsc, aop = p.aop;
   const bool need_y = vop_reads_y(vop);
   const bool use_val = (rop == ROP_NOOP) && (vsc != VSC_NOOP);
   const bool use_sop_udef = (p.sop == OP_UDEF);
   const int wpc = blockDim.x >> 5;
   long long wid = static_cast<long long>(blockIdx.x) * wpc + (threadIdx.x >> 5);
   const long long stride = static_cast<long long>(gridDim.x) * wpc;
   long long nh = 0, nchunks = 0;
   if (p.mode == MODE_HUB_CHUNKS) {
      grid_dependency_wait();
      const unsigned long long c = *p.counter;
      nh = static_cast<long long>(c >> HUB_SHIFT);
      nchunks = static_cast<long long>(c & HUB_CHUNK_MASK);
      if (nh > p.hub_cap || nchunks > p.chunk_cap) return;
   }
   for (;; wid += stride) {
      WorkItem w;
      if (p.mode == MODE_ROWS) {
         if (wid >= p.m) return;
         w.row = wid;
         w.eb = ld_index(p.pntrb, wid, p.ptr64);
         w.ee = ld_index(p.pntre, wid, p.ptr64);
         w.dst_item = -1;
         if (w.ee - w.eb > p.chunk) return;
      } else {
         if (wid >= nchunks) return;
         chunk_item(p, p.order ? __ldg(p.order + wid) : wid, nh, w);
      }
      const T *xr = p.x + w.row * p.ldx;  // dereferenced only when a stage reads X
      const bool to_z = w.dst_item < 0;
      const bool remote = !(p.skip_empty_remote && w.eb == w.ee);
      T *dst = to_z ? p.z + w.row * p.ldz : p.partials + w.dst_item * p.k;
      const bool need_x = vop_reads_x(vop) || rop_reads_x(rop);

      // One edge's scalar: the reduction over ALL of K (or a_uv), then the scalar function.
      auto edge_scalar = [&](long long j, const T *yr) -> T {
         T s;
         if (rop != ROP_NOOP) {
            // four independent partial sums: four loads of X and of Y in flight per lane instead of one
            T s4[4] = {T(0), T(0), T(0), T(0)};
            long long t = lane;
            for (; t + 96 < p.k; t += 128) {
               T xe[4], ye[4];
#pragma unroll
               for (int q = 0; q < 4; q++) {
                  xe[q] = need_x ? xr[t + 32 * q] : T(0);
                  ye[q] = need_y ? __ldg(yr + t + 32 * q) : T(0);
               }
#pragma unroll
               for (int q = 0; q < 4; q++) s4[q] += rop_term(rop, xe[q], vop_apply(vop, xe[q], ye[q]));
            }
            for (; t < p.k; t += 32) {
               const T xe = need_x ? xr[t] : T(0);
               const T ye = need_y ? __ldg(yr + t) : T(0);
               s4[0] += rop_term(rop, xe, vop_apply(vop, xe, ye));
            }
            s = (s4[0] + s4[1]) + (s4[2] + s4[3]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(FULL, s, off);
         } else {
            s = use_val ? __ldg(p.val + j) : T(0);
         }
         return use_sop_udef ? sop_udef(s, p.sop_kind, p.sp0, p.sp1, p.sp2, p.sop_table) : s;
      };
      // When K spans several tiles and the message has a reduction, every tile needs every edge's scalar again:
      // compute them once and keep them in shared memory (one per edge of the item) instead of walking all of K
      // once per tile and edge.
      extern __shared__ __align__(16) unsigned char any_smem[];  // blockDim.x / 32 * ANY_MAX_CACHED values
      T *mine = reinterpret_cast<T *>(any_smem) + (threadIdx.x >> 5) * ANY_MAX_CACHED;
      const bool cached = rop != ROP_NOOP && p.k > 32 * EPT && w.ee - w.eb <= ANY_MAX_CACHED;
      if (cached) {
         __syncwarp();  // the previous item's scalars are no longer read
         for (long long j = w.eb; j < w.ee; j++) {
            const long long cid = need_y ? ld_index(p.indx, j, p.idx64) : 0;
            const T out = edge_scalar(j, p.y + cid * p.ldy);
            if (lane == 0) mine[j - w.eb] = out;
         }
         __syncwarp();
      }

      for (long long kt = 0; kt < p.k; kt += 32 * EPT) {
         T acc[EPT];
#pragma unroll
         for (int e = 0; e < EPT; e++) acc[e] = aop_identity<T>(aop);
         for (long long j = w.eb; j < w.ee; j++) {
            const long long cid = need_y ? ld_index(p.indx, j, p.idx64) : 0;
            const T *yr = p.y + cid * p.ldy;
            const T out = cached ? mine[j - w.eb] : edge_scalar(j, yr);
#pragma unroll
            for (int e = 0; e < EPT; e++) {
               const long long t = kt + e * 32 + lane;
               if (t < p.k) {
                  const T xe = need_x ? xr[t] : T(0);
                  const T ye = need_y ? __ldg(yr + t) : T(0);
                  T tt = vop_apply(vop, xe, ye);
                  if (vsc == VSC_MUL) tt = out * tt;
                  else if (vsc == VSC_ADD) tt = out + tt;
                  acc[e] = aop_apply(aop, acc[e], tt);
               }
            }
         }
#pragma unroll
         for (int e = 0; e < EPT; e++) {
            const long long t = kt + e * 32 + lane;
            if (t < p.k) {
               T r = acc[e];
               if (to_z && p.accumulate) r = aop_apply(aop, dst[t], r);
               if (to_z && p.z_mc && remote) {
                  st_multicast(p.z_mc + w.row * p.ldz + t, r);
               } else {
                  dst[t] = r;
                  if (to_z && remote)
                     for (int q = 0; q < p.n_peers; q++) p.z_peer[q][w.row * p.ldz + t] = r;
               }
            }
         }
      }
      if (p.mode == MODE_ROWS) return;
   }
}

// ---------------------------------------------------------------------------------------------------
// Row scheduler, device side.
// ---------------------------------------------------------------------------------------------------
// Pass 1: find the rows that have more than `chunk` edges.  Each gets a slot in the hub list and a
// contiguous run of ceil(deg/chunk) chunk indices, both taken from ONE packed atomic so that
// hub_base[] is increasing in the slot number.
__global__ void scan_hub_rows(const void *pntrb, const void *pntre, int ptr64, long long m,
                              long long chunk, unsigned long long *counter, long long *hub_row,
                              long long *hub_base, long long hub_cap);

// Pass 3: for every split row, Z_row = AOP(old Z_row or identity, partial_0, partial_1, ...).
// Rows of up to FIXUP_LONG chunks: one warp per row, lanes strided over K, the chunks in order.  Longer rows (a row
// of 400 000 edges has 1 600 chunks, and a single warp adding them one after the other is the tail of the whole call):
// one block per row; warp w adds the w-th of blockDim.x/32 equal runs of consecutive chunks in order, then warp 0 adds
// Z_row and the runs' sums in run order.  The association of the additions depends only on the row's chunk count and
// the block size (fixed), so results are the same from run to run.
constexpr int FIXUP_LONG = 48;

template <typename T>
__device__ __forceinline__ void reduce_hub_row_block(const Params<T> &p, long long row, long long base, long long nch,
                                                     T (*seg)[128])
{
   constexpr int EPT = 4;
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
   const long long per = (nch + nw - 1) / nw;
   const long long q0 = warp * per, q1 = q0 + per < nch ? q0 + per : nch;
   T *zr = p.z + row * p.ldz;
   for (long long kt = 0; kt < p.k; kt += 32 * EPT) {
      T a[EPT];
#pragma unroll
      for (int e = 0; e < EPT; e++) a[e] = aop_identity<T>(p.aop);
      const T *src = p.partials + (base + q0) * p.k + kt + lane;
#pragma unroll 4
      for (long long q = q0; q < q1; q++, src += p.k) {
         T v[EPT];
#pragma unroll
         for (int e = 0; e < EPT; e++) v[e] = (kt + e * 32 + lane < p.k) ? __ldcg(src + e * 32) : aop_identity<T>(p.aop);
#pragma unroll
         for (int e = 0; e < EPT; e++) a[e] = aop_apply(p.aop, a[e], v[e]);
      }
#pragma unroll
      for (int e = 0; e < EPT; e++) seg[warp][e * 32 + lane] = a[e];
      __syncthreads();
      if (warp == 0) {
#pragma unroll
         for (int e = 0; e < EPT; e++) {
            const long long t = kt + e * 32 + lane;
            if (t < p.k) {
               T r = p.accumulate ? zr[t] : aop_identity<T>(p.aop);
               for (int w = 0; w < nw && w * per < nch; w++) r = aop_apply(p.aop, r, seg[w][e * 32 + lane]);
               if (p.z_mc) {
                  st_multicast(p.z_mc + row * p.ldz + t, r);
               } else {
                  zr[t] = r;
                  for (int g = 0; g < p.n_peers; g++) p.z_peer[g][row * p.ldz + t] = r;
               }
            }
         }
      }
      __syncthreads();
   }
}

template <typename T>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
hub_fixup_kernel(const Params<T> p)
{
   __shared__ T seg[WARPS_PER_CTA][128];
   __shared__ long long long_slot[WARPS_PER_CTA * 32];
   __shared__ int n_long;
   const int lane = threadIdx.x & 31;
   grid_dependency_wait();  // the partial sums come from the chunk launch that precedes this one
   const unsigned long long c = *p.counter;
   const long long nh = static_cast<long long>(c >> HUB_SHIFT);
   const long long nchunks = static_cast<long long>(c & HUB_CHUNK_MASK);
   if (nh > p.hub_cap || nchunks > p.chunk_cap) return;
   // the long rows first, so that they do not start last: every thread looks at one slot, the block then works through
   // the long ones it found.  Neighbouring slots (the longest rows of a skewed graph sit together) go to different blocks.
   for (long long s0 = 0; s0 < nh; s0 += static_cast<long long>(gridDim.x) * blockDim.x) {
      if (threadIdx.x == 0) n_long = 0;
      __syncthreads();
      const long long slot = s0 + static_cast<long long>(threadIdx.x) * gridDim.x + blockIdx.x;
      if (slot < nh) {
         const long long row = p.hub_row[slot];
         const long long deg = ld_index(p.pntre, row, p.ptr64) - ld_index(p.pntrb, row, p.ptr64);
         if ((deg + p.chunk - 1) / p.chunk > FIXUP_LONG) long_slot[atomicAdd(&n_long, 1)] = slot;
      }
      __syncthreads();
      const int n = n_long;
      for (int i = 0; i < n; i++) {
         const long long sl = long_slot[i];
         const long long row = p.hub_row[sl], base = p.hub_base[sl];
         const long long deg = ld_index(p.pntre, row, p.ptr64) - ld_index(p.pntrb, row, p.ptr64);
         reduce_hub_row_block(p, row, base, (deg + p.chunk - 1) / p.chunk, seg);
      }
      __syncthreads();
   }
   const int wpc = blockDim.x >> 5;
   const long long stride = static_cast<long long>(gridDim.x) * wpc;
   for (long long slot = static_cast<long long>(blockIdx.x) * wpc + (threadIdx.x >> 5); slot < nh;
        slot += stride) {
      const long long row = p.hub_row[slot], base = p.hub_base[slot];
      const long long deg = ld_index(p.pntre, row, p.ptr64) - ld_index(p.pntrb, row, p.ptr64);
      const long long nch = (deg + p.chunk - 1) / p.chunk;
      if (nch <= FIXUP_LONG) reduce_hub_row(p, row, base, nch, lane);
   }
}

// Z_row = 0 for every row without edges: what a call with beta == 0 leaves in such rows.  A GPU of a multi-GPU
// run does this to the rows of the OTHER GPUs' shards in its own copy of Z, so that those rows need not cross
// NVLink.  One warp per 32 rows: each lane looks at one row, then the warp zeroes the empty ones together.
template <typename T>
__global__ void __launch_bounds__(256)
zero_empty_rows_kernel(const void *pntrb, const void *pntre, int ptr64, long long m, long long k, T *z, long long ldz)
{
   const int lane = threadIdx.x & 31;
   const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
   const long long r = warp * 32 + lane;
   const bool empty = r < m && ld_index(pntre, r, ptr64) <= ld_index(pntrb, r, ptr64);
   unsigned mask = __ballot_sync(FULL, empty);
   const bool vec = (k % VecOf<T>::W == 0) && (ldz % VecOf<T>::W == 0) && ((reinterpret_cast<uintptr_t>(z) & 15) == 0);
   while (mask) {
      const int src = __ffs(mask) - 1;
      mask &= mask - 1;
      T *zr = z + (warp * 32 + src) * ldz;
      if (vec) {
         const T zero[VecOf<T>::W] = {};
         for (long long t = static_cast<long long>(lane) * VecOf<T>::W; t < k; t += 32 * VecOf<T>::W) st_vec(zr + t, zero);
      } else {
         for (long long t = lane; t < k; t += 32) zr[t] = T(0);
      }
   }
}

// ---------------------------------------------------------------------------------------------------
// Host-side launch table (defined in the per-pattern translation units).
// ---------------------------------------------------------------------------------------------------
enum : int { PAT_GENERIC = 0, PAT_SIGMOID = 1, PAT_TDIST = 2, PAT_SPMM = 3, PAT_GCN = 4 };
#ifndef __CUDACC_RTC__
// <<<grid, block, 0, stream>>> with, when p.pdl is set, the attribute that lets the kernel overlap its launch with
// the tail of the kernel before it in the stream.
template <typename T>
inline cudaError_t launch_kernel(void (*kern)(const Params<T>), long long grid, int threads, cudaStream_t stream, const Params<T> &p,
                                 size_t dynamic_smem = 0)
{
   cudaLaunchConfig_t cfg = {};
   cfg.gridDim = dim3(static_cast<unsigned int>(grid));
   cfg.blockDim = dim3(threads);
   cfg.dynamicSmemBytes = dynamic_smem;
   cfg.stream = stream;
   cudaLaunchAttribute attr[1];
   attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
   attr[0].val.programmaticStreamSerializationAllowed = 1;
   cfg.attrs = attr;
   cfg.numAttrs = p.pdl ? 1 : 0;
   return cudaLaunchKernelEx(&cfg, kern, p);
}

// Launches fused_vec_kernel<T, pattern ops, G, NV, U> with `grid` CTAs on `stream`.
// Returns false when that (G, NV) tiling is not instantiated.
template <typename T>
bool launch_vec(int pattern, int G, int NV, int U, int warps, const Params<T> &p, long long grid, cudaStream_t stream);
template <typename T>
void launch_any(const Params<T> &p, int warps, long long grid, cudaStream_t stream);
template <typename T>
void launch_fixup(const Params<T> &p, long long grid, cudaStream_t stream);

// Message-specific kernels built at run time (fusedmm_jit.cu): launches fused_vec_kernel<T, vop, rop, vsc, aop, G,
// NV, U, MB> compiled by NVRTC for exactly this message.  Returns false when there is no such kernel (NVRTC not
// found, compilation failed, the policy says this message is not worth compiling yet): the caller then launches the
// flag-interpreting instantiation.  `weight` is the size of the call (edges x K, 0 if unknown) for that policy.
template <typename T>
bool jit_launch_vec(int vop, int rop, int vsc, int aop, int G, int NV, int U, int MB, int flags, int warps, const Params<T> &p,
                    long long grid, cudaStream_t stream, int policy, long long weight);
// Compile (or find in the cache) without launching; 0 on success.  Works without a GPU.
int jit_prepare(int is_double, int vop, int rop, int vsc, int aop, int G, int NV, int U, int MB, int flags);
struct JitStats { long long compiled, disk_hits, launches, failures; int nvrtc_found; };
JitStats jit_stats();
#endif

}  // namespace fmm
