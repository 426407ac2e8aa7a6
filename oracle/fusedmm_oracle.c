/*
 * CPU oracle for fusedMM_csr -- TEST INFRASTRUCTURE ONLY.
 *
 * Only the tests, the smoke check and the benchmark's CPU-baseline leg may load this.  The product
 * (libfusedmm_b200.so) never links, loads or calls it and has no CPU path of its own.
 *
 * Parity status: PINNED.  The reference has no golden vectors, so the pin is the reference itself:
 * oracle/build_ref.sh compiles HipGraph/FusedMM's own fusedMM.c, and tests/test_oracle_pin.py
 * requires this restatement to equal it bit for bit on seeded inputs; tests/golden/ holds outputs of
 * that reference build for machines without the reference sources.
 *
 * The algorithm is in fusedmm_oracle_body.inc (included once per type combination below); this
 * file adds the scalar functions a caller of the reference would link as SOP_UDEF_FUNC.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "sop_bodies.h"

/* evaluate one scalar function: lets the tests pin the SOP bodies on their own */
float  oracle_sop_f32(float s, int kind, double p0, double p1, double p2) { return or_sop_f(s, kind, p0, p1, p2); }
double oracle_sop_f64(double s, int kind, double p0, double p1, double p2) { return or_sop_d(s, kind, p0, p1, p2); }

/* ---- instantiations -------------------------------------------------------------------------------- */
#define OR_VT float
#define OR_PT int32_t
#define OR_IT int32_t
#define OR_SOP or_sop_f
#define OR_NAME oracle_sfusedMM_csr_i32
#include "fusedmm_oracle_body.inc"

#define OR_VT float
#define OR_PT int64_t
#define OR_IT int64_t
#define OR_SOP or_sop_f
#define OR_NAME oracle_sfusedMM_csr_i64
#include "fusedmm_oracle_body.inc"

#define OR_VT float
#define OR_PT int64_t
#define OR_IT int32_t
#define OR_SOP or_sop_f
#define OR_NAME oracle_sfusedMM_csr_p64i32
#include "fusedmm_oracle_body.inc"

#define OR_VT double
#define OR_PT int32_t
#define OR_IT int32_t
#define OR_SOP or_sop_d
#define OR_NAME oracle_dfusedMM_csr_i32
#include "fusedmm_oracle_body.inc"

#define OR_VT double
#define OR_PT int64_t
#define OR_IT int64_t
#define OR_SOP or_sop_d
#define OR_NAME oracle_dfusedMM_csr_i64
#include "fusedmm_oracle_body.inc"

#define OR_VT double
#define OR_PT int64_t
#define OR_IT int32_t
#define OR_SOP or_sop_d
#define OR_NAME oracle_dfusedMM_csr_p64i32
#include "fusedmm_oracle_body.inc"
