/*
 * Harness linked with the UNMODIFIED reference sources -- TEST INFRASTRUCTURE ONLY.
 *
 * oracle/build_ref.sh compiles <reference>/fusedMM.c once per (VALUETYPE, INDEXTYPE) together with
 * this file into oracle/_ref/libfusedmm_ref_<s|d>_<i32|i64>.so.  The harness supplies what a caller
 * of the reference must supply: the SOP_UDEF_FUNC body (fusedMM.h:131,139) and the thread count.
 * Exports:
 *    ref_fusedMM_csr   the reference's fusedMM_csr (fusedMM.c:487-744), re-exported unchanged
 *    ref_set_sop       choose which scalar function SOP_UDEF_FUNC evaluates
 *    ref_set_threads   team size used by the reference's `omp_set_num_threads(NTHREADS)`
 */
#include <omp.h>
#include <stdint.h>
#ifdef DREAL
#define VALUETYPE double
#define REF_SOP or_sop_d
#else
#define VALUETYPE float
#define REF_SOP or_sop_f
#endif
#include "fusedMM.h" /* the reference's header, found through -I<reference> */
#include "sop_bodies.h"

static int    g_kind = 1;
static double g_p0 = 0, g_p1 = 0, g_p2 = 0;
static int    g_threads = 0;

void ref_set_sop(int kind, double p0, double p1, double p2) { g_kind = kind; g_p0 = p0; g_p1 = p1; g_p2 = p2; }
void ref_set_threads(int n) { g_threads = n; }
int  fusedmm_ref_nthreads(void) { return g_threads > 0 ? g_threads : omp_get_num_procs(); }
int  ref_get_threads(void) { return fusedmm_ref_nthreads(); }

int SOP_UDEF_FUNC(VALUETYPE val, VALUETYPE *out)
{
   *out = REF_SOP(val, g_kind, g_p0, g_p1, g_p2);
   return FUSEDMM_SUCCESS_RETURN;
}

int ref_fusedMM_csr(const int32_t imessage, const INDEXTYPE m, const INDEXTYPE n, const INDEXTYPE k,
                    const VALUETYPE alpha, const INDEXTYPE nnz, const INDEXTYPE rows,
                    const INDEXTYPE cols, const VALUETYPE *val, const INDEXTYPE *indx,
                    const INDEXTYPE *pntrb, const INDEXTYPE *pntre, const VALUETYPE *x,
                    const INDEXTYPE ldx, const VALUETYPE *y, const INDEXTYPE ldy, const VALUETYPE beta,
                    VALUETYPE *z, const INDEXTYPE ldz)
{
   return fusedMM_csr(imessage, m, n, k, alpha, nnz, rows, cols, val, indx, pntrb, pntre, x, ldx, y,
                      ldy, beta, z, ldz);
}
