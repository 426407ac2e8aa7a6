/*
 * kernels.h -- source-compatible replacement for kernels/include/kernels.h of HipGraph/FusedMM: the
 * second public entry of the reference, its optimised-kernel dispatcher, backed by libfusedmm_b200.so.
 *
 * Usage is the reference's: define INDEXTYPE (int32_t | int64_t) before including this file and call
 *
 *    sgfusedMM_csr(tkern, m, n, k, alpha, nnz, rows, cols, val, indx, pntrb, pntre,
 *                  A, lda, B, ldb, beta, C, ldc);           (dgfusedMM_csr for double)
 *
 * with tkern = 't' (t-distribution / FR), 's' (sigmoid), 'm' (SpMM) or 'g' (GCN), as declared at
 * kernels/include/kernels.h:17-43 and defined at kernels/src/kernels.c:456-631 there.  The reference
 * compiles those two names once per INDEXTYPE; a shared library cannot export two ABIs under one name, so
 * the names below are macros that forward to the typed symbols {s,d}gfusedMM_csr_{i32,i64} of
 * include/fusedmm_b200.h chosen from the caller's INDEXTYPE.  trusted_{s,d}gfusedMM_csr, the reference's
 * scalar fallbacks (kernels.c:45-453), forward to the same symbols: the GPU library has one
 * implementation for every K.
 *
 * The scalar function behind 't' and 's': the reference's generated kernels call the SOP_UDEF_FUNC the
 * program links (genkern.base:113,122,487,554).  When VALUETYPE is defined before this header is included
 * (as every caller of fusedMM.h does), the program's SOP_UDEF_FUNC, if it defines one, is handed to the
 * library, which evaluates it on the host at sample points to find the built-in device function it equals
 * (fusedmm_b200.h, FUSEDMM_SOP_*).  Otherwise the process-wide default applies (fusedmm_b200_set_sop).
 */
#ifndef FUSEDMM_B200_DROPIN_KERNELS_H
#define FUSEDMM_B200_DROPIN_KERNELS_H

#include <stdint.h>
#include "fusedmm_b200.h"

#ifndef INDEXTYPE
#error "define INDEXTYPE as int32_t or int64_t before including kernels.h"
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define FUSEDMM_B200_KERNELS_IS_I64 (sizeof(INDEXTYPE) == sizeof(int64_t))

#ifdef VALUETYPE
/* weak: a program without the hook still links (same declaration as in fusedMM.h) */
int SOP_UDEF_FUNC(VALUETYPE val, VALUETYPE *out) __attribute__((weak));
#define FUSEDMM_B200_KERNELS_HOOK(VT) \
   (sizeof(VALUETYPE) == sizeof(VT) ? (int (*)(VT, VT *))(void (*)(void))SOP_UDEF_FUNC : (int (*)(VT, VT *))0)
#else
#define FUSEDMM_B200_KERNELS_HOOK(VT) ((int (*)(VT, VT *))0)
#endif

/* The casts are no-ops on the branch that is taken; the other branch is dead code that only has to compile. */
#define FUSEDMM_B200_DEFINE_G_DROPIN(NAME, VT, PRE)                                                      \
   static inline void NAME(const char tkern, const INDEXTYPE m, const INDEXTYPE n, const INDEXTYPE k,   \
                           const VT alpha, const INDEXTYPE nnz, const INDEXTYPE rows,                   \
                           const INDEXTYPE cols, const VT *val, const INDEXTYPE *indx,                  \
                           const INDEXTYPE *pntrb, const INDEXTYPE *pntre, const VT *A,                 \
                           const INDEXTYPE lda, const VT *B, const INDEXTYPE ldb, const VT beta, VT *C, \
                           const INDEXTYPE ldc)                                                         \
   {                                                                                                    \
      if (FUSEDMM_B200_KERNELS_IS_I64)                                                                  \
         PRE##gfusedMM_csr_i64_udef(tkern, (int64_t)m, (int64_t)n, (int64_t)k, alpha, (int64_t)nnz,          \
                               (int64_t)rows, (int64_t)cols, val, (const int64_t *)(const void *)indx,  \
                               (const int64_t *)(const void *)pntrb,                                    \
                               (const int64_t *)(const void *)pntre, A, (int64_t)lda, B, (int64_t)ldb,  \
                               beta, C, (int64_t)ldc, FUSEDMM_B200_KERNELS_HOOK(VT));                   \
      else                                                                                              \
         PRE##gfusedMM_csr_i32_udef(tkern, (int32_t)m, (int32_t)n, (int32_t)k, alpha, (int32_t)nnz,          \
                               (int32_t)rows, (int32_t)cols, val, (const int32_t *)(const void *)indx,  \
                               (const int32_t *)(const void *)pntrb,                                    \
                               (const int32_t *)(const void *)pntre, A, (int32_t)lda, B, (int32_t)ldb,  \
                               beta, C, (int32_t)ldc, FUSEDMM_B200_KERNELS_HOOK(VT));                   \
   }

FUSEDMM_B200_DEFINE_G_DROPIN(sgfusedMM_csr_b200_dropin, float, s)
FUSEDMM_B200_DEFINE_G_DROPIN(dgfusedMM_csr_b200_dropin, double, d)

#define sgfusedMM_csr          sgfusedMM_csr_b200_dropin
#define dgfusedMM_csr          dgfusedMM_csr_b200_dropin
#define trusted_sgfusedMM_csr  sgfusedMM_csr_b200_dropin
#define trusted_dgfusedMM_csr  dgfusedMM_csr_b200_dropin

#ifdef __cplusplus
}
#endif
#endif /* FUSEDMM_B200_DROPIN_KERNELS_H */
