/*
 * fusedMM.h -- source-compatible replacement for the header of HipGraph/FusedMM, backed by
 * libfusedmm_b200.so (hand-written sm_100a CUDA kernels).
 *
 * Usage is the reference's: define VALUETYPE (float | double) and INDEXTYPE (int32_t | int64_t)
 * before including this file (usually -DINDEXTYPE=int64_t on the compiler line), build a message
 * out of one flag per stage, and call
 *
 *    fusedMM_csr(imessage, m, n, k, alpha, nnz, rows, cols, val, indx, pntrb, pntre,
 *                x, ldx, y, ldy, beta, z, ldz);
 *
 * The flag names and values below are the wire format of `imessage` and therefore identical to
 * the reference's (fusedMM.h:18-73 there).  fusedMM_csr here is a macro that forwards to the typed
 * symbol of libfusedmm_b200.so that matches VALUETYPE and INDEXTYPE and hands it the address of the
 * caller's SOP_UDEF_FUNC, if the program defines one.
 */
#ifndef FUSEDMM_B200_DROPIN_FUSEDMM_H
#define FUSEDMM_B200_DROPIN_FUSEDMM_H

#include <stdint.h>
#include "fusedmm_b200.h"

#ifndef VALUETYPE
#error "define VALUETYPE as float or double before including fusedMM.h"
#endif
#ifndef INDEXTYPE
#error "define INDEXTYPE as int32_t or int64_t before including fusedMM.h"
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- stage 1, VOP: T = op(X_u, Y_v); nibble 0 ------------------------------------------------ */
#define FUSEDMM_NIBBLE(code, pos) (((int32_t)(code)) << (4 * (pos)))
#define VOP_NOOP      FUSEDMM_NIBBLE(0x0, 0)
#define VOP_COPY_LHS  FUSEDMM_NIBBLE(0x1, 0)   /* T = X_u                                        */
#define VOP_COPY_RHS  FUSEDMM_NIBBLE(0x2, 0)   /* T = Y_v                                        */
#define VOP_ADD       FUSEDMM_NIBBLE(0x3, 0)   /* T = X_u + Y_v                                  */
#define VOP_SUBL      FUSEDMM_NIBBLE(0x4, 0)   /* T = Y_v - X_u  (what the reference computes)   */
#define VOP_SUBR      FUSEDMM_NIBBLE(0x5, 0)   /* T = X_u - Y_v  (what the reference computes)   */
#define VOP_MAX       FUSEDMM_NIBBLE(0x6, 0)
#define VOP_MIN       FUSEDMM_NIBBLE(0x7, 0)
#define VOP_UDEF      FUSEDMM_NIBBLE(0xF, 0)
/* ---- stage 2, ROP: s = reduce(X_u, T); nibble 1 ---------------------------------------------- */
#define ROP_NOOP      FUSEDMM_NIBBLE(0x0, 1)   /* s = a_uv                                       */
#define ROP_DOT       FUSEDMM_NIBBLE(0x1, 1)
#define ROP_ADD_LHS   FUSEDMM_NIBBLE(0x2, 1)
#define ROP_ADD_RHS   FUSEDMM_NIBBLE(0x3, 1)
#define ROP_NORML     FUSEDMM_NIBBLE(0x4, 1)
#define ROP_NORMR     FUSEDMM_NIBBLE(0x5, 1)
#define ROP_UDEF      FUSEDMM_NIBBLE(0xF, 1)
/* ---- stage 3, SOP: out = f(s); nibble 2 ------------------------------------------------------ */
#define SOP_NOOP      FUSEDMM_NIBBLE(0x0, 2)
#define SOP_COPY      FUSEDMM_NIBBLE(0x1, 2)
#define SOP_UDEF      FUSEDMM_NIBBLE(0xF, 2)
/* ---- stage 4, VSC (MOP): T = out (*|+) T; nibble 3 ------------------------------------------- */
#define VSC_NOOP      FUSEDMM_NIBBLE(0x0, 3)
#define VSC_MUL       FUSEDMM_NIBBLE(0x1, 3)
#define VSC_ADD       FUSEDMM_NIBBLE(0x2, 3)
#define VSC_UDEF      FUSEDMM_NIBBLE(0xF, 3)
/* ---- stage 5, AOP: Z_u = acc(Z_u, T); nibble 4 ----------------------------------------------- */
#define AOP_NOOP      FUSEDMM_NIBBLE(0x0, 4)
#define AOP_ADD       FUSEDMM_NIBBLE(0x1, 4)
#define AOP_MAX       FUSEDMM_NIBBLE(0x2, 4)
#define AOP_MIN       FUSEDMM_NIBBLE(0x3, 4)
#define AOP_UDEF      FUSEDMM_NIBBLE(0xF, 4)

/* get / set / clear helpers with the reference's names */
#define FUSEDMM_FIELD(pos)        FUSEDMM_NIBBLE(0xF, pos)
#define VOP_MASK(bvec)            ((bvec) & FUSEDMM_FIELD(0))
#define ROP_MASK(bvec)            ((bvec) & FUSEDMM_FIELD(1))
#define SOP_MASK(bvec)            ((bvec) & FUSEDMM_FIELD(2))
#define VSC_MASK(bvec)            ((bvec) & FUSEDMM_FIELD(3))
#define AOP_MASK(bvec)            ((bvec) & FUSEDMM_FIELD(4))
#define VOP_CLEAR(bvec)           ((bvec) & ~FUSEDMM_FIELD(0))
#define ROP_CLEAR(bvec)           ((bvec) & ~FUSEDMM_FIELD(1))
#define SOP_CLEAR(bvec)           ((bvec) & ~FUSEDMM_FIELD(2))
#define VSC_CLEAR(bvec)           ((bvec) & ~FUSEDMM_FIELD(3))
#define AOP_CLEAR(bvec)           ((bvec) & ~FUSEDMM_FIELD(4))
#define GET_VOP_FLAG(imsg)        VOP_MASK(imsg)
#define GET_ROP_FLAG(imsg)        ROP_MASK(imsg)
#define GET_SOP_FLAG(imsg)        SOP_MASK(imsg)
#define GET_VSC_FLAG(imsg)        VSC_MASK(imsg)
#define GET_AOP_FLAG(imsg)        AOP_MASK(imsg)
#define SET_VOP_FLAG(imsg, f)     ((imsg) = (VOP_CLEAR(imsg) | (f)))
#define SET_ROP_FLAG(imsg, f)     ((imsg) = (ROP_CLEAR(imsg) | (f)))
#define SET_SOP_FLAG(imsg, f)     ((imsg) = (SOP_CLEAR(imsg) | (f)))
#define SET_VSC_FLAG(imsg, f)     ((imsg) = (VSC_CLEAR(imsg) | (f)))
#define SET_AOP_FLAG(imsg, f)     ((imsg) = (AOP_CLEAR(imsg) | (f)))

/* return codes, reference names */
#define FUSEDMM_SUCCESS_RETURN            FUSEDMM_B200_OK
#define FUSEDMM_FAIL_RETURN               1
#define FUSEDMM_VOP_FAIL_RETURN           FUSEDMM_B200_ERR_VOP
#define FUSEDMM_ROP_FAIL_RETURN           FUSEDMM_B200_ERR_ROP
#define FUSEDMM_AOP_FAIL_RETURN           FUSEDMM_B200_ERR_AOP
#define FUSEDMM_SOP_FAIL_RETURN           FUSEDMM_B200_ERR_SOP
#define FUSEDMM_VSC_FAIL_RETURN           FUSEDMM_B200_ERR_VSC
#define FUSEDMM_NOT_ENOUGH_MEM            FUSEDMM_B200_ERR_NOMEM
#define FUSEDMM_UNDEFINED_USER_FUNCTION   FUSEDMM_B200_ERR_UDEF
#define FUSEDMM_NO_OPT_IMPL               FUSEDMM_B200_ERR_NO_OPT

/*
 * User hook.  Only the scalar stage can be user defined here, and only when its body is one of the
 * functions the device knows (fusedmm_b200.h, FUSEDMM_SOP_*): the hook is a host function and is
 * evaluated on the host at a few sample points to find out which one it is.  The declaration is weak
 * so that a program without the hook still links; SOP_UDEF then means the process-wide default.
 * VOP/ROP/VSC/AOP user functions cannot run on the GPU: those messages return
 * FUSEDMM_UNDEFINED_USER_FUNCTION.
 */
int SOP_UDEF_FUNC(VALUETYPE val, VALUETYPE *out) __attribute__((weak));
/* The other four hooks, with the reference's signatures (fusedMM.h:135-143 there), so that a program that
 * defines one with a different signature is diagnosed at compile time as it would be against the
 * reference's header.  They are never called: a kernel cannot run host code. */
int VOP_UDEF_FUNC(INDEXTYPE lhs_dim, const VALUETYPE *lhs, INDEXTYPE rhs_dim, const VALUETYPE *rhs,
                  INDEXTYPE out_dim, VALUETYPE *out);
int ROP_UDEF_FUNC(INDEXTYPE lhs_dim, const VALUETYPE *lhs, INDEXTYPE rhs_dim, const VALUETYPE *rhs,
                  VALUETYPE *out);
int VSC_UDEF_FUNC(INDEXTYPE rhs_dim, const VALUETYPE *rhs, VALUETYPE scal, INDEXTYPE out_dim,
                  VALUETYPE *out);
int AOP_UDEF_FUNC(INDEXTYPE rhs_dim, const VALUETYPE *rhs, INDEXTYPE out_dim, VALUETYPE *out);

/* compile-time choice of the typed symbol */
#define FUSEDMM_B200_IS_DOUBLE   (sizeof(VALUETYPE) == sizeof(double))
#define FUSEDMM_B200_IS_I64      (sizeof(INDEXTYPE) == sizeof(int64_t))

static inline int fusedMM_csr_b200_dropin(
   const int32_t imessage, const INDEXTYPE m, const INDEXTYPE n, const INDEXTYPE k,
   const VALUETYPE alpha, const INDEXTYPE nnz, const INDEXTYPE rows, const INDEXTYPE cols,
   const VALUETYPE *val, const INDEXTYPE *indx, const INDEXTYPE *pntrb, const INDEXTYPE *pntre,
   const VALUETYPE *x, const INDEXTYPE ldx, const VALUETYPE *y, const INDEXTYPE ldy,
   const VALUETYPE beta, VALUETYPE *z, const INDEXTYPE ldz)
{
   /* The casts are no-ops on the branch that is taken; the other branches are dead code that only
    * has to compile. */
   if (FUSEDMM_B200_IS_DOUBLE) {
      int (*hook)(double, double *) = (int (*)(double, double *))(void (*)(void))SOP_UDEF_FUNC;
      if (FUSEDMM_B200_IS_I64)
         return dfusedMM_csr_i64_udef(imessage, m, n, k, (double)alpha, nnz, rows, cols,
               (const double *)(const void *)val, (const int64_t *)(const void *)indx,
               (const int64_t *)(const void *)pntrb, (const int64_t *)(const void *)pntre,
               (const double *)(const void *)x, ldx, (const double *)(const void *)y, ldy,
               (double)beta, (double *)(void *)z, ldz, hook);
      return dfusedMM_csr_i32_udef(imessage, (int32_t)m, (int32_t)n, (int32_t)k, (double)alpha,
            (int32_t)nnz, (int32_t)rows, (int32_t)cols, (const double *)(const void *)val,
            (const int32_t *)(const void *)indx, (const int32_t *)(const void *)pntrb,
            (const int32_t *)(const void *)pntre, (const double *)(const void *)x, (int32_t)ldx,
            (const double *)(const void *)y, (int32_t)ldy, (double)beta, (double *)(void *)z,
            (int32_t)ldz, hook);
   } else {
      int (*hook)(float, float *) = (int (*)(float, float *))(void (*)(void))SOP_UDEF_FUNC;
      if (FUSEDMM_B200_IS_I64)
         return sfusedMM_csr_i64_udef(imessage, m, n, k, (float)alpha, nnz, rows, cols,
               (const float *)(const void *)val, (const int64_t *)(const void *)indx,
               (const int64_t *)(const void *)pntrb, (const int64_t *)(const void *)pntre,
               (const float *)(const void *)x, ldx, (const float *)(const void *)y, ldy,
               (float)beta, (float *)(void *)z, ldz, hook);
      return sfusedMM_csr_i32_udef(imessage, (int32_t)m, (int32_t)n, (int32_t)k, (float)alpha,
            (int32_t)nnz, (int32_t)rows, (int32_t)cols, (const float *)(const void *)val,
            (const int32_t *)(const void *)indx, (const int32_t *)(const void *)pntrb,
            (const int32_t *)(const void *)pntre, (const float *)(const void *)x, (int32_t)ldx,
            (const float *)(const void *)y, (int32_t)ldy, (float)beta, (float *)(void *)z,
            (int32_t)ldz, hook);
   }
}
#define fusedMM_csr fusedMM_csr_b200_dropin

#ifdef __cplusplus
}
#endif
#endif /* FUSEDMM_B200_DROPIN_FUSEDMM_H */
