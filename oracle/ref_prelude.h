/*
 * Force-included (gcc -include) in front of the reference's own fusedMM.c when oracle/build_ref.sh
 * compiles it -- TEST INFRASTRUCTURE ONLY.  The reference hard-codes its OpenMP team size as the
 * macro NTHREADS (fusedMM.c:634, set at configure time, configure:276-286); the build recipe defines
 * NTHREADS as a call of this function so that one binary uses the cores of whatever host runs it.
 */
#ifndef FUSEDMM_REF_PRELUDE_H
#define FUSEDMM_REF_PRELUDE_H
int fusedmm_ref_nthreads(void);
#endif
