/*
 * fusedmm_b200.h -- C ABI of libfusedmm_b200.so
 *
 * A from-scratch sm_100a (NVIDIA B200) implementation of the FusedMM operation
 *
 *     Z_u  =  AOP_v ( VSC( SOP( ROP( X_u, VOP(X_u, Y_v) ) or a_uv ), VOP(X_u, Y_v) ) )   for every edge (u,v) of a CSR matrix
 *
 * behind the entry point of HipGraph/FusedMM.  Every function below is `extern "C"`, takes plain
 * pointers and integer sizes and no CUDA or torch types, so that C host code (and cgo / JNI / ctypes
 * bindings) can call it.  Each declaration cites the reference interface it replaces as
 * `file:line` inside the HipGraph/FusedMM source tree.
 *
 * Pointer residency.  The reference only sees host memory.  Here every array argument may
 * independently be a device pointer (used in place, nothing is copied) or a host pointer (staged to the
 * GPU for the call; Z is copied back before the call returns).  Residency is detected per pointer
 * with cudaPointerGetAttributes.  Unless stated otherwise a call is synchronous: Z is complete when
 * it returns, exactly like the reference; when it is given device arrays it first waits for all work
 * already enqueued on the device (cudaDeviceSynchronize), because it runs on a stream of its own.
 *
 * Threads.  Every entry point may be called from any host thread.  Calls that target the same device (the
 * device that is current in the calling thread) run one after the other; calls from different threads on
 * DIFFERENT devices run side by side, so one process can drive several GPUs (one thread per GPU, each with its
 * own device current and its row shard).  Options and the default SOP are process-wide; a call uses the values
 * in force when it starts.
 *
 * There is no CPU implementation in this library.  If no CUDA device is usable every entry point
 * returns FUSEDMM_B200_ERR_CUDA.
 */
#ifndef FUSEDMM_B200_H
#define FUSEDMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------
 * Status codes.  Non-negative values are the reference's (fusedMM.h:103-112) and keep their
 * meaning; negative values below -1 are new and report CUDA-side failures.
 * ---------------------------------------------------------------------------------------------- */
#define FUSEDMM_B200_OK                  0    /* FUSEDMM_SUCCESS_RETURN            fusedMM.h:103 */
#define FUSEDMM_B200_ERR_VOP             2    /* FUSEDMM_VOP_FAIL_RETURN           fusedMM.h:105 */
#define FUSEDMM_B200_ERR_ROP             4    /* FUSEDMM_ROP_FAIL_RETURN           fusedMM.h:106 */
#define FUSEDMM_B200_ERR_AOP             8    /* FUSEDMM_AOP_FAIL_RETURN           fusedMM.h:107 */
#define FUSEDMM_B200_ERR_SOP             16   /* FUSEDMM_SOP_FAIL_RETURN           fusedMM.h:108 */
#define FUSEDMM_B200_ERR_VSC             32   /* FUSEDMM_VSC_FAIL_RETURN           fusedMM.h:109 */
#define FUSEDMM_B200_ERR_NOMEM          (-1)  /* FUSEDMM_NOT_ENOUGH_MEM            fusedMM.h:110 */
#define FUSEDMM_B200_ERR_UDEF            64   /* FUSEDMM_UNDEFINED_USER_FUNCTION   fusedMM.h:111 */
#define FUSEDMM_B200_ERR_NO_OPT          128  /* FUSEDMM_NO_OPT_IMPL               fusedMM.h:112 */
#define FUSEDMM_B200_ERR_CUDA           (-2)  /* a CUDA runtime call failed, or no device            */
#define FUSEDMM_B200_ERR_ARG            (-3)  /* negative size, ld < k, null pointer that is needed  */
#define FUSEDMM_B200_ERR_LIMIT          (-4)  /* a fixed capacity was exceeded (see the entry point) */

/* ------------------------------------------------------------------------------------------------
 * Scalar operations (SOP) that can run on the device.
 *
 * The reference resolves SOP_UDEF to a host function `int SOP_UDEF_FUNC(VALUETYPE, VALUETYPE*)`
 * linked by the caller (fusedMM.h:139) and calls it once per edge (fusedMM.c:729).  A GPU kernel
 * cannot call a host function, so the bodies the reference's own tester links
 * (test/fusedMMtime.cpp:625-674) plus the two that the benchmark configurations name are built in.
 * Which one SOP_UDEF means is chosen, in this order, by
 *   1. an explicit `fusedmm_b200_sop` passed to fusedmm_b200_csr();
 *   2. a host SOP_UDEF_FUNC pointer passed to a *_udef entry point: it is evaluated on the host at a
 *      fixed set of sample points and matched against the built-ins (no match -> status 64; see option
 *      "strict_udef" for the limits of that match);
 *   3. the process-wide default set with fusedmm_b200_set_sop() (initially SIGMOID).
 * ---------------------------------------------------------------------------------------------- */
#define FUSEDMM_SOP_IDENTITY        0  /* out = s                      default body, fusedMMtime.cpp:669-673 */
#define FUSEDMM_SOP_SIGMOID         1  /* out = 1/(1+exp(-s))                                               */
#define FUSEDMM_SOP_SIGMOID_TABLE_C 2  /* out = 1 - table_sigmoid(s)   fusedMMtime.cpp:586-611, :628-632     */
#define FUSEDMM_SOP_FR              3  /* out = 1 + 1/s                fusedMMtime.cpp:635-639               */
#define FUSEDMM_SOP_TDIST           4  /* out = 1/(1+s)                                                     */
#define FUSEDMM_SOP_TDIST_CLAMPED   5  /* out = clamp(-2/(1+s), +-5)   fusedMMtime.cpp:612-617, :642-646     */
#define FUSEDMM_SOP_LL              6  /* out = log2(1+sqrt(s))        fusedMMtime.cpp:649-653               */
#define FUSEDMM_SOP_FA              7  /* out = sqrt(s) + 1/s          fusedMMtime.cpp:656-660               */
#define FUSEDMM_SOP_AFFINE_RECIP    8  /* out = clamp(p0/(p1+s), +-p2) when p2>0, else p0/(p1+s)            */
#define FUSEDMM_SOP_KIND_COUNT      9

typedef struct fusedmm_b200_sop {
   int32_t kind;      /* one of FUSEDMM_SOP_*                                  */
   int32_t reserved;  /* must be 0                                             */
   double  p0, p1, p2;/* parameters of FUSEDMM_SOP_AFFINE_RECIP, else ignored  */
} fusedmm_b200_sop;

int fusedmm_b200_set_sop(int32_t kind, double p0, double p1, double p2);
int fusedmm_b200_get_sop(fusedmm_b200_sop *out);

/* ------------------------------------------------------------------------------------------------
 * fusedMM_csr, one symbol per (VALUETYPE, INDEXTYPE) build of the reference.
 *
 * Replaces: int fusedMM_csr(imessage, m, n, k, alpha, nnz, rows, cols, val, indx, pntrb, pntre,
 *                           x, ldx, y, ldy, beta, z, ldz)        fusedMM.h:76-97, fusedMM.c:487-744
 * Argument meaning, order and the return codes are the reference's.  As in the reference `alpha`,
 * `n`, `nnz`, `rows` and `cols` are not read; `m` rows are processed.  `beta == 0` overwrites Z (rows
 * without edges become 0), any other beta accumulates into Z, which is the behaviour of the
 * reference's optimised kernels (kernels/src/kernels.c:501-520); see fusedmm_b200_set_option
 * ("beta_mode") for the general kernel's behaviour.
 *
 * The reference compiles one function named fusedMM_csr per choice of the VALUETYPE and INDEXTYPE
 * macros; a shared library cannot export four ABIs under one name, so the symbols carry the types
 * (s|d = float|double, i32|i64 = INDEXTYPE) and include/fusedMM.h maps the reference's name onto
 * the one that matches the caller's macros.
 * ---------------------------------------------------------------------------------------------- */
#define FUSEDMM_B200_DECL_CSR(NAME, VT, IT)                                                        \
   int NAME(const int32_t imessage, const IT m, const IT n, const IT k, const VT alpha,            \
            const IT nnz, const IT rows, const IT cols, const VT *val, const IT *indx,             \
            const IT *pntrb, const IT *pntre, const VT *x, const IT ldx, const VT *y,              \
            const IT ldy, const VT beta, VT *z, const IT ldz)

FUSEDMM_B200_DECL_CSR(sfusedMM_csr_i32, float,  int32_t);
FUSEDMM_B200_DECL_CSR(sfusedMM_csr_i64, float,  int64_t);
FUSEDMM_B200_DECL_CSR(dfusedMM_csr_i32, double, int32_t);
FUSEDMM_B200_DECL_CSR(dfusedMM_csr_i64, double, int64_t);

/* The reference's default build (VALUETYPE float, INDEXTYPE int64_t; kernels/CONFIG/make.base:151,155)
 * is also exported under the reference's own symbol name `fusedMM_csr`, for objects that were
 * compiled against the reference's header with exactly those types and are only re-linked.  It is
 * declared here on request only, because include/fusedMM.h defines that name as a macro. */
#if defined(FUSEDMM_B200_DECLARE_REFERENCE_SYMBOL) && !defined(fusedMM_csr)
FUSEDMM_B200_DECL_CSR(fusedMM_csr, float, int64_t);
#endif

/* Same call with the caller's host SOP_UDEF_FUNC (fusedMM.h:139) handed over explicitly; used by
 * the fusedMM_csr wrapper of include/fusedMM.h.  `sop_udef` may be NULL. */
#define FUSEDMM_B200_DECL_CSR_UDEF(NAME, VT, IT)                                                   \
   int NAME(const int32_t imessage, const IT m, const IT n, const IT k, const VT alpha,            \
            const IT nnz, const IT rows, const IT cols, const VT *val, const IT *indx,             \
            const IT *pntrb, const IT *pntre, const VT *x, const IT ldx, const VT *y,              \
            const IT ldy, const VT beta, VT *z, const IT ldz, int (*sop_udef)(VT, VT *))

FUSEDMM_B200_DECL_CSR_UDEF(sfusedMM_csr_i32_udef, float,  int32_t);
FUSEDMM_B200_DECL_CSR_UDEF(sfusedMM_csr_i64_udef, float,  int64_t);
FUSEDMM_B200_DECL_CSR_UDEF(dfusedMM_csr_i32_udef, double, int32_t);
FUSEDMM_B200_DECL_CSR_UDEF(dfusedMM_csr_i64_udef, double, int64_t);

/* Mixed index widths: 64-bit row pointers and sizes with 32-bit column ids.  The reference has a
 * single INDEXTYPE (fusedMM.h:79-96) and cannot express this; it is what a graph with more than
 * 2^31 edges but fewer than 2^31 vertices wants. */
int sfusedMM_csr_p64i32(const int32_t imessage, const int64_t m, const int64_t n, const int64_t k,
                        const float alpha, const int64_t nnz, const int64_t rows, const int64_t cols,
                        const float *val, const int32_t *indx, const int64_t *pntrb,
                        const int64_t *pntre, const float *x, const int64_t ldx, const float *y,
                        const int64_t ldy, const float beta, float *z, const int64_t ldz);
int dfusedMM_csr_p64i32(const int32_t imessage, const int64_t m, const int64_t n, const int64_t k,
                        const double alpha, const int64_t nnz, const int64_t rows, const int64_t cols,
                        const double *val, const int32_t *indx, const int64_t *pntrb,
                        const int64_t *pntre, const double *x, const int64_t ldx, const double *y,
                        const int64_t ldy, const double beta, double *z, const int64_t ldz);

/* ------------------------------------------------------------------------------------------------
 * The optimised-kernel dispatcher, callable directly.
 * Replaces: void sgfusedMM_csr / dgfusedMM_csr (const char tkern, ...)   kernels/include/kernels.h:17-37,
 *           kernels/src/kernels.c:456-631.   tkern: 't' t-dist/FR, 's' sigmoid, 'm' SpMM, 'g' GCN.
 * Like the reference they return nothing; an unknown letter prints a message to stderr.  The SOP for
 * 't' and 's' is the process-wide default (fusedmm_b200_set_sop).
 * ---------------------------------------------------------------------------------------------- */
#define FUSEDMM_B200_DECL_G(NAME, VT, IT)                                                          \
   void NAME(const char tkern, const IT m, const IT n, const IT k, const VT alpha, const IT nnz,   \
             const IT rows, const IT cols, const VT *val, const IT *indx, const IT *pntrb,         \
             const IT *pntre, const VT *A, const IT lda, const VT *B, const IT ldb, const VT beta, \
             VT *C, const IT ldc)

FUSEDMM_B200_DECL_G(sgfusedMM_csr_i32, float,  int32_t);
FUSEDMM_B200_DECL_G(sgfusedMM_csr_i64, float,  int64_t);
FUSEDMM_B200_DECL_G(dgfusedMM_csr_i32, double, int32_t);
FUSEDMM_B200_DECL_G(dgfusedMM_csr_i64, double, int64_t);

/* Same dispatcher with the caller's host SOP_UDEF_FUNC handed over explicitly (the reference's generated
 * kernels call the hook the program links: kernels/codegen/genkern.base:113,122,487,554); used by the
 * {s,d}gfusedMM_csr wrappers of include/kernels.h.  `sop_udef` may be NULL (process-wide default). */
#define FUSEDMM_B200_DECL_G_UDEF(NAME, VT, IT)                                                     \
   void NAME(const char tkern, const IT m, const IT n, const IT k, const VT alpha, const IT nnz,   \
             const IT rows, const IT cols, const VT *val, const IT *indx, const IT *pntrb,         \
             const IT *pntre, const VT *A, const IT lda, const VT *B, const IT ldb, const VT beta, \
             VT *C, const IT ldc, int (*sop_udef)(VT, VT *))

FUSEDMM_B200_DECL_G_UDEF(sgfusedMM_csr_i32_udef, float,  int32_t);
FUSEDMM_B200_DECL_G_UDEF(sgfusedMM_csr_i64_udef, float,  int64_t);
FUSEDMM_B200_DECL_G_UDEF(dgfusedMM_csr_i32_udef, double, int32_t);
FUSEDMM_B200_DECL_G_UDEF(dgfusedMM_csr_i64_udef, double, int64_t);

/* ------------------------------------------------------------------------------------------------
 * The one function all of the above funnel into.
 *
 *   dtype     0 = float, 1 = double                       (VALUETYPE, fusedMM.c:9-13)
 *   ptr_bits  32 or 64: width of pntrb / pntre entries
 *   idx_bits  32 or 64: width of indx entries             (INDEXTYPE, fusedMM.h:79-96)
 *   sop       NULL = process-wide default
 *   stream    NULL = run on the library's own stream and return when Z is complete.
 *             Otherwise a cudaStream_t: all work is enqueued on it and the call returns without
 *             waiting; every array must then be a device pointer (else FUSEDMM_B200_ERR_ARG), and
 *             a capacity overflow of the split-row scratch (only possible when nnz understates the
 *             graph: a positive nnz sizes the scratch before the launches) is reported by
 *             fusedmm_b200_stream_status().  The scratch is per device: calls enqueued on different
 *             streams of one device must be ordered by the caller.
 * Everything else: as fusedMM_csr (fusedMM.h:76-97).
 * ---------------------------------------------------------------------------------------------- */
int fusedmm_b200_csr(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage,
                     int64_t m, int64_t n, int64_t k, double alpha, int64_t nnz, int64_t rows,
                     int64_t cols, const void *val, const void *indx, const void *pntrb,
                     const void *pntre, const void *x, int64_t ldx, const void *y, int64_t ldy,
                     double beta, void *z, int64_t ldz, const fusedmm_b200_sop *sop, void *stream);

/* ------------------------------------------------------------------------------------------------
 * fusedmm_b200_csr with the Z exchange of a multi-GPU run fused into the kernels: every finished row
 * of Z is stored into `z` and, with the same layout (same ldz, same row numbering), into each of the
 * n_peers (<= 8) buffers z_peers[i], which are device addresses of OTHER GPUs' Z buffers that this
 * GPU can write (peer-mapped memory, e.g. the buffer_ptrs of a torch symmetric-memory tensor, offset
 * to this call's first row).  The stores are plain global stores that cross NVLink; nothing is read
 * from a peer.  The caller orders the ranks: a peer's rows are complete in this GPU's Z once that peer's
 * call has finished (stream order on the peer) and a cross-rank barrier or collective has been passed.
 * z_multicast, when not NULL, replaces the peer list: it is the address, at this call's first row, of
 * an NVSwitch multicast mapping of Z (it covers this GPU's copy too); each finished row is then stored
 * once with multimem.st and the switch delivers it to every GPU, so a rank sends its rows once, not
 * once per peer.  No counterpart in the reference (which is single-process, fusedMM.c:487-744).
 *
 * Rows without edges are NOT sent (option "multi_skip_empty_rows", default 1): their result is a constant
 * that every GPU can produce itself from the row pointers it already holds, and on R-MAT graphs they are a
 * quarter to half of all rows.  The call stores such a row (zeros when beta == 0, the unchanged Z_u otherwise)
 * into this GPU's `z` only.  The other GPUs bring their own copies up to date with
 * fusedmm_b200_zero_empty_rows over the rows of the foreign shards when beta == 0; with beta != 0 there is
 * nothing to do as long as every GPU's Z held the same values on entry.
 * ---------------------------------------------------------------------------------------------- */
int fusedmm_b200_csr_multi(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage,
                           int64_t m, int64_t n, int64_t k, double alpha, int64_t nnz, int64_t rows,
                           int64_t cols, const void *val, const void *indx, const void *pntrb,
                           const void *pntre, const void *x, int64_t ldx, const void *y, int64_t ldy,
                           double beta, void *z, int64_t ldz, const fusedmm_b200_sop *sop, void *stream,
                           int32_t n_peers, void *const *z_peers, void *z_multicast);

/* Z_u = 0 for every row u < m with pntre[u] <= pntrb[u], on `stream` (NULL: the default stream, and the call
 * waits): what fusedMM_csr with beta == 0 leaves in rows without edges (kernels/codegen/genkern.base:287-295).
 * Device arrays only.  Used by the GPUs of a multi-GPU run on the rows of the other GPUs' shards (see
 * fusedmm_b200_csr_multi).  No counterpart in the reference. */
int fusedmm_b200_zero_empty_rows(int32_t dtype, int32_t ptr_bits, int64_t m, int64_t k, const void *pntrb,
                                 const void *pntre, void *z, int64_t ldz, void *stream);

/* ------------------------------------------------------------------------------------------------
 * fusedmm_b200_csr for callers that must not allocate.
 *
 * Some hosts of this library may not touch the CUDA allocator once they are running: a serving
 * process that gave all device memory to its own pool at start-up and would simply get
 * out-of-memory from cudaMalloc; a real-time loop for which cudaMalloc/cudaFree are off limits
 * because they may synchronise the whole device and stall every other stream; a plugin sandbox that
 * is only allowed to launch kernels.  The other entry points keep their split-row scratch (hub list,
 * per-chunk partial sums) in buffers they cudaMalloc and grow on demand, and create a stream and
 * events on first use.  This one calls no cudaMalloc, cudaFree, stream/event creation or any other
 * allocating routine: the same kernels run with their scratch inside a fixed 32 MiB array that is
 * part of the library image (every GPU the library runs on holds that array from load to exit).
 *
 * Same arguments and results as fusedmm_b200_csr, with these limits:
 *   - every array must already be in device memory (FUSEDMM_B200_ERR_ARG otherwise);
 *   - nnz must be the true number of edges of the m rows: it is what bounds the scratch. The call is
 *     refused with FUSEDMM_B200_ERR_LIMIT and a message on stderr when
 *     nnz/c + 1 > 32768 (split rows) or 2*(nnz/c) + 1 partial rows of k values do not fit in the
 *     array, c = max(512, option hub_chunk) being the edges per piece this entry point uses, e.g. more
 *     than about 16.4 million edges at k = 128 floats;
 *   - all launches go to `stream`, or to the legacy default stream when stream is NULL, in which case
 *     the call returns after they have finished;
 *   - the first call on a device looks up the array's address on that device and copies the two 2048-entry
 *     sigmoid tables (float and double) into it with two small synchronous copies; later calls copy
 *     nothing.  Make that first call outside any stream capture;
 *   - with a non-NULL stream the call returns without waiting; if nnz understated the graph, the split rows
 *     of that call are not computed and fusedmm_b200_stream_status(), called after the stream's work has
 *     completed, returns FUSEDMM_B200_ERR_LIMIT for it (with a truthful nnz this cannot happen);
 *   - the array is shared by all calls on a device and keeps the previous call's contents (the call
 *     clears the one word that has to start at zero); two calls whose kernels may overlap on the GPU
 *     (different streams without an ordering between them) race on it and must not be issued.
 * It has no counterpart in the reference, whose only scratch is a K-element array on each thread's
 * stack.
 * ---------------------------------------------------------------------------------------------- */
int fusedmm_b200_csr_static_scratch(int32_t dtype, int32_t ptr_bits, int32_t idx_bits, int32_t imessage,
                                    int64_t m, int64_t n, int64_t k, double alpha, int64_t nnz,
                                    int64_t rows, int64_t cols, const void *val, const void *indx,
                                    const void *pntrb, const void *pntre, const void *x, int64_t ldx,
                                    const void *y, int64_t ldy, double beta, void *z, int64_t ldz,
                                    const fusedmm_b200_sop *sop, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Inspector / executor split for callers that run many messages over one fixed graph (the epochs of
 * an embedding or GNN training loop).  The reference redoes its row partition in every thread on every
 * call (fusedMM.c:633-676) and its timers anticipate "an inspector phase" (test/fusedMMtime.cpp:1483-1485).
 *
 * fusedmm_b200_plan_create copies host CSR arrays to the current device once (device arrays are
 * borrowed: keep them alive and unchanged while the plan lives), finds the rows that have to be split and
 * keeps that list; for large graphs it also sorts the pieces of the split rows by column and the other rows by
 * length inside windows (options "chunk_order", "row_bins": the values in force when the plan is made).  val may be NULL (val_dtype ignored) for graphs used only with messages that do not
 * read edge values; val_dtype: 0 float, 1 double.  nnz is ignored (the extent is the largest row end).
 * fusedmm_b200_plan_csr is fusedmm_b200_csr without the CSR arguments: x, y, z may be host or device
 * arrays, stream as in fusedmm_b200_csr.  Per call it saves the scan and the sort launches (three launches instead
 * of eight on a large graph) and, for host callers, the copy of the column ids and edge values.  A plan belongs to the device it was created on.
 * ---------------------------------------------------------------------------------------------- */
typedef struct fusedmm_b200_plan fusedmm_b200_plan;
int fusedmm_b200_plan_create(int32_t ptr_bits, int32_t idx_bits, int64_t m, int64_t nnz, const void *indx,
                             const void *pntrb, const void *pntre, int32_t val_dtype, const void *val,
                             fusedmm_b200_plan **out);
int fusedmm_b200_plan_csr(const fusedmm_b200_plan *plan, int32_t dtype, int32_t imessage, int64_t n, int64_t k,
                          const void *x, int64_t ldx, const void *y, int64_t ldy, double beta, void *z,
                          int64_t ldz, const fusedmm_b200_sop *sop, void *stream);
int fusedmm_b200_plan_destroy(fusedmm_b200_plan *plan);

/* After work enqueued with a non-NULL stream has completed: 0, or FUSEDMM_B200_ERR_LIMIT when the
 * hub-row scratch was too small for that call.  The rows with at most hub_chunk edges have then been
 * computed and the longer rows have not been touched; the scratch has been enlarged.  Running the call
 * again gives the right Z when the call overwrites Z (beta == 0 on the four optimised messages).  A call
 * that accumulates (beta != 0, or any other message) has already added its short rows' contributions:
 * restore Z before running it again.  A positive, truthful nnz sizes the scratch before the launches, so
 * the case only arises when nnz understates the graph or is 0. */
int fusedmm_b200_stream_status(void);

/* ------------------------------------------------------------------------------------------------
 * Row scheduler pieces that are useful on their own.
 *
 * fusedmm_b200_shard_rows_*: cut rows [0,m) into `nshards` contiguous ranges of (nearly) equal edge
 * count: bounds[g] .. bounds[g+1] is shard g, bounds has nshards+1 entries.  This lifts the idea of
 * the reference's per-thread partition (fusedMM.c:633-676; rows are never split) from OpenMP threads
 * to GPUs.  pntrb/pntre are HOST pointers here.  A shard is then computed with an ordinary
 * fusedMM_csr call on (m = bounds[g+1]-bounds[g], pntrb + bounds[g], pntre + bounds[g],
 * x + bounds[g]*ldx, z + bounds[g]*ldz): the four-array CSR needs no re-basing.
 * ---------------------------------------------------------------------------------------------- */
int fusedmm_b200_shard_rows_i32(int64_t m, int32_t nshards, const int32_t *pntrb,
                                const int32_t *pntre, int64_t *bounds);
int fusedmm_b200_shard_rows_i64(int64_t m, int32_t nshards, const int64_t *pntrb,
                                const int64_t *pntre, int64_t *bounds);
/* The same with a fixed cost per row added to its edge count (row_weight >= 0, in edges): a row also costs a
 * read of X_u, a write of Z_u and, between GPUs, the transfer of Z_u, whatever its degree.  0 gives the
 * functions above. */
int fusedmm_b200_shard_rows_weighted_i32(int64_t m, int32_t nshards, const int32_t *pntrb,
                                         const int32_t *pntre, int64_t row_weight, int64_t *bounds);
int fusedmm_b200_shard_rows_weighted_i64(int64_t m, int32_t nshards, const int64_t *pntrb,
                                         const int64_t *pntre, int64_t row_weight, int64_t *bounds);

/* ------------------------------------------------------------------------------------------------
 * Validates a CSR on the GPU before it is trusted (the kernels themselves do not bounds-check, like
 * the reference: fusedMM.c:706-712).  report[0] = rows with pntre < pntrb or pntrb < 0, report[1] =
 * column ids outside [0, n), report[2] = edges of the m rows, report[3] = largest degree.  Returns 0,
 * or FUSEDMM_B200_ERR_ARG when report[0] or report[1] is not zero.  Host or device arrays.
 * No counterpart in the reference (its -DDEBUG build only compares vector dimensions, fusedMM.c:31-37).
 * ---------------------------------------------------------------------------------------------- */
int fusedmm_b200_check_csr(int32_t ptr_bits, int32_t idx_bits, int64_t m, int64_t n, const void *indx,
                           const void *pntrb, const void *pntre, int64_t *report);

/* ------------------------------------------------------------------------------------------------
 * Options, introspection, teardown.
 *
 * fusedmm_b200_set_option(name, value) -> 0, or FUSEDMM_B200_ERR_ARG for an unknown name/value:
 *   "beta_mode"      0 (default): the four patterns the reference has optimised kernels for honour
 *                    beta (0 = overwrite) and every other message accumulates into Z, i.e. a build of
 *                    the reference with ENABLE_OPT_FUSEDMM (fusedMM.c:512-605);
 *                    1: every message accumulates into Z whatever beta is, i.e. the reference's
 *                    general kernel (fusedMM.c:698-739).
 *   "accept_vop_noop" 0 (default): VOP_NOOP returns status 2 as in the reference (fusedMM.c:346-377);
 *                    1: VOP_NOOP means T = Y_v.
 *   "hub_chunk"      most edges a row may have before it is split across warps, and edges per piece
 *                    (default 256; a call whose nnz argument is below 2^24 uses at most 128, below 2^21
 *                    at most 64, unless a row of k values exceeds 1024 bytes).
 *   "chunk_ctas_per_sm"  blocks per SM of the launch that works on the pieces of split rows (default 3).
 *   "chunk_order"        the pieces of split rows are visited sorted by the column id of their first edge (a counting
 *                        sort on the device: three more launches per call, none with a plan, which sorts once), so that
 *                        the pieces in flight at one time gather from one band of Y: 0 never, 1 (default) for graphs of
 *                        16 M edges and more (judged by the nnz argument, or 16 x m when that is 0), 2 always.  Results
 *                        do not depend on it.
 *   "force_tiling"   0 = automatic; otherwise (register_budget << 24) | (gathers_in_flight << 16) |
 *                    (lanes_per_edge << 8) | vectors_per_lane; gathers_in_flight 0 means that tiling's
 *                    default, register_budget 0 the compiler's choice (only instantiated combinations
 *                    are accepted, see fusedmm_b200/csrc/fusedmm_inst.cuh).
 *   "warps_per_cta"  1..8 (default 1): block size of the main kernel, in warps.
 *   "engine"         0 or 1 (default): the row scheduler (a warp per row, long rows cut into chunks);
 *                    2: the edge-stream scheduler (equal-sized edge quanta, rows split where the
 *                    quanta end) whenever pntre == pntrb + 1 entry and the 16-byte vector path applies.
 *   "edge_quantum"   edges per work item of the edge-stream scheduler (default 256; rounded up to a
 *                    multiple of 32).
 *   "stream_depth"   neighbour rows each group of lanes keeps in flight in shared memory (default 16;
 *                    rounded down to a power of two, at least 8 or the lanes per edge if fewer).
 *   "side_priority"  1 (default): the stream that carries the chunks of split rows has the device's greatest
 *                    priority, so their blocks are placed before the whole-row launch's when both are pending
 *                    (3-8 % faster on a B200); 0: default priority.
 *   "side_stream"    1 (default): the chunks of split rows run on a second stream beside the whole rows;
 *                    0: every launch on one stream (12 % slower on the benchmark graph; diagnostic).
 *   "force_tiling_rows"  as force_tiling, for the whole-row launch only (0 = the call's tiling).
 *   "force_generic"  1 = run every message through the flag-interpreting kernel; 2 = treat the four built-in
 *                    patterns like any other message (flag-interpreting kernel, or a run-time-built one as option
 *                    "jit" decides): diagnostics.
 *   "jit"            what a message outside the four built-in patterns runs on.  The reference has optimised
 *                    kernels for four messages and a function-pointer loop for the rest (fusedMM.c:512-605,
 *                    :698-739; its TODO :516-518 asks for generated kernels for "all vector ops").  Here the
 *                    kernel template is instantiated for the message at hand at run time with NVRTC, cached in
 *                    the process and as a cubin under $FUSEDMM_B200_JIT_CACHE (default ~/.cache/fusedmm_b200;
 *                    empty = no files).  1 (default): build it once the same message and K class has been
 *                    launched 16 times (8 calls), or at once when nnz * k >= 2^26 (about a second, once per
 *                    machine); until then, and if NVRTC (libnvrtc.so.12, or $FUSEDMM_B200_NVRTC) is missing, the
 *                    flag-interpreting kernel runs, which is 1.7-2.2x slower.  0: never build.  2: build on first
 *                    use.  fusedmm_b200_jit_prepare builds ahead of time.
 *   "pdl"            1 (default): the chain scan -> chunks of split rows -> fix-up is launched with programmatic
 *                    stream serialization, so each kernel becomes resident while its predecessor drains (what
 *                    matters for small graphs, where launch gaps are a tenth of the call); 0: plain launches.
 *   "timing_detail"  1 (default): a synchronous call records an event after each launch (the ms_* fields of
 *                    fusedmm_b200_call_info); those records sit between the kernels of the chain and undo "pdl"
 *                    for that call.  0: only ms_main and device_ms are measured, the launches stay paired.
 *   "multi_skip_empty_rows"  1 (default): fusedmm_b200_csr_multi does not send rows without edges to the other
 *                    GPUs (see there); 0: every row of the shard is sent.
 *   "strict_udef"    0 (default): a host SOP_UDEF_FUNC handed to a *_udef entry point is evaluated at 25 sample
 *                    points and replaced by the built-in device function that equals it there (none: status 64);
 *                    a function that differs from the built-in only between or beyond the sample points is not
 *                    told apart.  1: such a hook is not examined and the call returns status 64; SOP_UDEF then
 *                    needs fusedmm_b200_set_sop or an explicit sop argument.
 *   "exact_k"        1 (default): a call whose k fills its tiling exactly (every power of two from 16 to 2048 floats,
 *                    8 to 1024 doubles) runs the instantiation without per-vector bounds predicates (7 % faster at
 *                    k = 256 floats, neutral at 128 and 512; bit-identical results); 0: always the general one.
 *   "element_vectors"  1 (default): a call whose k, leading dimensions or base addresses are not multiples of 16 bytes
 *                    and whose k is at most 512 runs the vector engine with one-element vectors (4- or 8-byte
 *                    accesses); 0: such calls take the element-strided engine, as rows longer than 512 elements do.
 *   "bulk_chunks"    0 (default): the chunks of split rows gather neighbour rows with per-lane 16-byte loads; 16 or 32:
 *                    with bulk asynchronous copies into a shared-memory ring of that many rows per warp
 *                    (fusedmm_b200/csrc/fusedmm_bulk.cuh; the four optimised messages only).  Same results; measured
 *                    15 % to 2.4x slower on the benchmark configurations.  "bulk_warps" (1..8, default 8): warps per
 *                    block of that launch; "bulk_ctas_per_sm" (0 = as many as fit).
 *   "blocked_inputs" 1 (default): in a call whose Z (32 MB or more) goes back to a host array block of rows by block of rows,
 *                    host column ids and edge values given with (rowptr, rowptr + 1) row pointers come in block by block
 *                    as well, behind the dense inputs, while earlier blocks compute and go out; 0: all inputs first.
 *   "offset32"       1 (default): with 32-bit column ids and rows of Y less than 2^32 bytes apart, the whole-row launch
 *                    of calls with 68..128 floats (34..64 doubles) per row runs the instantiation that forms a neighbour
 *                    row's address with one 32 x 32 + 64-bit multiply-add (bit-identical results; 4 % faster at
 *                    k = 128 floats; the other tilings measured slower with it and have no such form); 0: never.
 *   "jit_call_shape" 0 (default); 1: a call with nnz * k >= 2^26 of ANY message runs a kernel built at run time for
 *                    the shape of the call (exact k, 32-bit column ids) in BOTH launches; 2: every call does.
 *                    Bit-identical results; an experiment, left off.
 *   "jit_shape_mask" bit 1 switches the 32-bit column ids of "jit_call_shape" on (default 3).
 *   "hub_cap_initial"  split rows the hub list has room for when it is first allocated (default 65536; it grows on
 *                    demand, this only sets where the growth starts: tests use it to reach the growth path).
 *   "inject_alloc_failure"  n > 0: the n-th device allocation the library attempts from now on fails
 *                    with FUSEDMM_B200_ERR_NOMEM (host-side fault injection for tests; nothing is
 *                    done to the GPU).
 * fusedmm_b200_get_option(name, &value) reads them back.
 * Environment: FUSEDMM_B200_OPTIONS="name=value,name=value" sets options when the library is loaded (for
 * programs that cannot be changed to call fusedmm_b200_set_option); FUSEDMM_B200_TRACE (any value) prints one line per call to stderr: message, sizes,
 * engine and tiling, launches, split rows, bytes copied and the CUDA-event times of the launches.
 * ---------------------------------------------------------------------------------------------- */
int fusedmm_b200_set_option(const char *name, int64_t value);
int fusedmm_b200_get_option(const char *name, int64_t *value);

/* Kernels launched / bytes copied by the most recent call on the calling thread. */
typedef struct fusedmm_b200_call_info {
   int32_t kernel_launches;   /* CUDA kernels of this library launched by the call           */
   int32_t pattern;           /* 0 generic, 1 sigmoid-like, 2 tdist/FR-like, 3 SpMM, 4 GCN   */
   int32_t lanes_per_edge;    /* tiling that was chosen; 0 = element-strided fallback        */
   int32_t vectors_per_lane;
   int64_t h2d_bytes;         /* staged host->device bytes                                   */
   int64_t d2h_bytes;         /* device->host bytes (Z)                                      */
   int64_t hub_rows;          /* row scheduler: rows split across several warps              */
   int64_t hub_chunks;        /* row scheduler: partial-row work items; edge stream: quanta  */
   float   device_ms;         /* CUDA-event time of the kernels of a synchronous call        */
   int32_t sop_kind;          /* SOP that ran                                                */
   /* CUDA-event time of each launch of a synchronous call, in launch order */
   float   ms_scan;           /* scan_hub_rows: finds the rows to split (from the start of the call) */
   float   ms_rows;           /* main kernel, one warp per whole row                         */
   float   ms_chunks;         /* main kernel over the chunks of split rows                   */
   float   ms_fixup;          /* hub_fixup_kernel: adds the chunk partials into Z            */
   int32_t engine;            /* 1 = row scheduler, 2 = edge-stream scheduler                */
   float   ms_main;           /* from the first launch of the call to the end of its last one: the whole-row
                                 launch runs beside the chain scan -> chunks -> fix-up             */
   int32_t jit_kernel;        /* 1: the main kernel was one built at run time for this message */
} fusedmm_b200_call_info;
int fusedmm_b200_last_call_info(fusedmm_b200_call_info *out);

/* Builds (or finds in the cache) the kernel specialised for `imessage` at feature length k and value type
 * dtype (0 float, 1 double) without running anything, so that the first real call does not pay for the
 * compilation; needs no GPU.  0 on success or when the message needs no such kernel (built-in pattern,
 * k not a multiple of 16 bytes); FUSEDMM_B200_ERR_NO_OPT when NVRTC is missing or the build failed; the
 * reference's status codes for an invalid message.  No counterpart in the reference, whose kernels are
 * generated at build time (kernels/CONFIG/rungen.top).
 * fusedmm_b200_jit_stats: out[0..4] = kernels compiled by this process, found in the file cache, launches of
 * run-time-built kernels, failures, NVRTC found (0/1). */
int fusedmm_b200_jit_prepare(int32_t dtype, int32_t imessage, int64_t k);
int fusedmm_b200_jit_stats(int64_t *out);

const char *fusedmm_b200_status_string(int status);
const char *fusedmm_b200_version(void);

/* Frees every device buffer the library holds (staging copies, hub-row scratch). */
int fusedmm_b200_release(void);

#ifdef __cplusplus
}
#endif
#endif /* FUSEDMM_B200_H */
