/*
 * Scalar (SOP) functions a caller of the reference links as SOP_UDEF_FUNC -- TEST INFRASTRUCTURE ONLY.
 * Shared by the CPU oracle (fusedmm_oracle.c) and by the harness that is compiled together with the
 * reference's own fusedMM.c (ref_harness.c), because in the reference these bodies are caller code,
 * not library code (fusedMM.h:139; the shipped bodies are in test/fusedMMtime.cpp:586-674).
 * The expressions follow C's promotion rules: literals are double, the result is rounded to the value
 * type once (the in-library C version of the table is kernels/codegen/genheader.base:43-61).
 */
#ifndef FUSEDMM_ORACLE_SOP_BODIES_H
#define FUSEDMM_ORACLE_SOP_BODIES_H
#include <math.h>
#include <stdint.h>

/*
 * Constants: SM_TABLE_SIZE 2048, SM_BOUND 5.0, SM_RESOLUTION = SM_TABLE_SIZE/(2.0*SM_BOUND)
 * (test/fusedMMtime.cpp:128-130).  Arithmetic on literals is double and the result is rounded to the
 * value type on assignment, as C does for the reference's expressions. */
#define OR_SM_SIZE 2048
#define OR_SM_BOUND 5.0

static float  or_table_f[OR_SM_SIZE];
static double or_table_d[OR_SM_SIZE];
static int    or_table_ready = 0;

/* uinit_SM_TABLE, test/fusedMMtime.cpp:595-604: x is stored in the value type before exp(). */
static void or_init_tables(void)
{
   if (or_table_ready) return;
   for (int i = 0; i < OR_SM_SIZE; i++) {
      float  xf = (float)(2.0 * OR_SM_BOUND * i / OR_SM_SIZE - OR_SM_BOUND);
      double xd = 2.0 * OR_SM_BOUND * i / OR_SM_SIZE - OR_SM_BOUND;
      or_table_f[i] = (float)(1.0 / (1 + exp(-xf)));
      or_table_d[i] = 1.0 / (1 + exp(-xd));
   }
   or_table_ready = 1;
}
__attribute__((constructor)) static void or_ctor(void) { or_init_tables(); }

/* The table index of ufast_SM (test/fusedMMtime.cpp:606-611).  v == SM_BOUND indexes one past the
 * table in the reference; the oracle (and the device code) clamp that single point to the last entry. */
static inline int or_table_index(double v)
{
   int idx = (int)((v + OR_SM_BOUND) * OR_SM_SIZE / (2.0 * OR_SM_BOUND));
   return idx > OR_SM_SIZE - 1 ? OR_SM_SIZE - 1 : idx;
}

#define OR_DEFINE_SOP(NAME, VT, TABLE)                                                             \
   static inline VT NAME(VT s, int kind, double p0, double p1, double p2)                          \
   {                                                                                               \
      switch (kind) {                                                                              \
         case 1: return (VT)(1.0 / (1.0 + exp(-(double)s)));          /* exact sigmoid          */ \
         case 2: {                                                    /* fusedMMtime.cpp:628-632 */ \
            VT sm;                                                                                 \
            if (s > OR_SM_BOUND) sm = (VT)1.0;                                                     \
            else if (s < -OR_SM_BOUND) sm = (VT)0.0;                                               \
            else sm = TABLE[or_table_index((double)s)];                                            \
            return (VT)(1.0 - sm);                                                                 \
         }                                                                                         \
         case 3: return (VT)(1.0 + 1.0 / s);                          /* fusedMMtime.cpp:635-639 */ \
         case 4: return (VT)(1.0 / (1.0 + s));                                                     \
         case 5: {                                                    /* fusedMMtime.cpp:642-646 */ \
            VT v = (VT)(-2.0 / (1.0 + s));                                                         \
            if (v > OR_SM_BOUND) return (VT)OR_SM_BOUND;                                           \
            if (v < -OR_SM_BOUND) return (VT)-OR_SM_BOUND;                                         \
            return v;                                                                              \
         }                                                                                         \
         case 6: return (VT)log2(1 + sqrt(s));                        /* fusedMMtime.cpp:649-653 */ \
         case 7: return (VT)(sqrt(s) + 1.0 / s);                      /* fusedMMtime.cpp:656-660 */ \
         case 8: {                                                                                 \
            VT v = (VT)(p0 / (p1 + s));                                                            \
            if (p2 > 0) { if (v > p2) v = (VT)p2; if (v < -p2) v = (VT)-p2; }                      \
            return v;                                                                              \
         }                                                                                         \
         default: return s;                                           /* fusedMMtime.cpp:669-673 */ \
      }                                                                                            \
   }
OR_DEFINE_SOP(or_sop_f, float, or_table_f)
OR_DEFINE_SOP(or_sop_d, double, or_table_d)

#endif
