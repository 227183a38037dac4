/* df32_ops.h -- double-float ("df32") arithmetic restated from the textbook
 * error-free transforms (Knuth TwoSum, Dekker FastTwoSum, FMA TwoProd).
 * TEST INFRASTRUCTURE ONLY (part of the CPU oracle).
 *
 * The reference takes these operations from the external metal-runtime project
 * (its df32 prelude: df_add / df_sub / df_mul / df_from_float / df_to_float, used
 * at examples/05_df32_precision.py:28-30,56-78), which is not in the reference
 * tree and has no pinned version: PARITY UNPINNED for the arithmetic in this
 * file.  Shared by oracle.c and by the build of the reference's own df32 kernel
 * text (msl_df32_ref.cpp), so both run the same operations.
 * Compile with -ffp-contract=off: every statement is one IEEE operation. */
#ifndef ORACLE_DF32_OPS_H_
#define ORACLE_DF32_OPS_H_
#include <math.h>

typedef struct { float hi, lo; } df;

static inline df two_sum(float a, float b) {          /* Knuth */
    df r; r.hi = a + b;
    float bv = r.hi - a;
    float av = r.hi - bv;
    r.lo = (a - av) + (b - bv);
    return r;
}
static inline df quick_two_sum(float a, float b) {    /* Dekker, |a| >= |b| */
    df r; r.hi = a + b; r.lo = b - (r.hi - a); return r;
}
static inline df two_prod(float a, float b) {         /* FMA */
    df r; r.hi = a * b; r.lo = fmaf(a, b, -r.hi); return r;
}
static inline df dfc(float a) { df r; r.hi = a; r.lo = 0.0f; return r; }
static inline df df_add(df a, df b) {
    df s = two_sum(a.hi, b.hi), t = two_sum(a.lo, b.lo);
    s.lo = s.lo + t.hi;
    s = quick_two_sum(s.hi, s.lo);
    s.lo = s.lo + t.lo;
    return quick_two_sum(s.hi, s.lo);
}
static inline df df_neg(df a) { df r; r.hi = -a.hi; r.lo = -a.lo; return r; }
static inline df df_sub(df a, df b) { return df_add(a, df_neg(b)); }
static inline df df_mul(df a, df b) {
    df p = two_prod(a.hi, b.hi);
    p.lo = fmaf(a.hi, b.lo, p.lo);
    p.lo = fmaf(a.lo, b.hi, p.lo);
    return quick_two_sum(p.hi, p.lo);
}
static inline df df_div(df a, df b) {
    float q1 = a.hi / b.hi;
    df r = df_sub(a, df_mul(dfc(q1), b));
    float q2 = r.hi / b.hi;
    r = df_sub(r, df_mul(dfc(q2), b));
    float q3 = r.hi / b.hi;
    return df_add(quick_two_sum(q1, q2), dfc(q3));
}
/* 1 / b: q = 1 / b.hi, e = 1 - b q formed exactly, result q + q e */
static inline df df_recip(df b) {
    float q = 1.0f / b.hi;
    df p = two_prod(b.hi, q);
    p.lo = fmaf(b.lo, q, p.lo);
    float e = (1.0f - p.hi) - p.lo;
    return quick_two_sum(q, q * e);
}
static inline df df_twice(df a) { df r; r.hi = a.hi + a.hi; r.lo = a.lo + a.lo; return r; }
static inline df df_sqrt(df a) {
    float s = sqrtf(a.hi);
    if (s == 0.0f) return dfc(0.0f);
    df d = df_sub(a, two_prod(s, s));
    return quick_two_sum(s, d.hi / (s + s));
}
/* 1 / sqrt(a), a > 0: integer seed, three float Newton steps, one second-order correction in df32 */
static inline df df_rsqrt(df a) {
    union { float f; unsigned u; } bits;
    float half_a = 0.5f * a.hi, y, e;
    df t;
    int i;
    bits.f = a.hi;
    bits.u = 0x5F375A86u - (bits.u >> 1);
    y = bits.f;
    for (i = 0; i < 3; ++i) {
        float yy = y * y;
        float h = half_a * yy;
        y = y * (1.5f - h);
    }
    t = df_mul(a, two_prod(y, y));
    e = (1.0f - t.hi) - t.lo;
    e = fmaf(0.75f * e, e, e);                       /* second-order term of (1 - e)^(-1/2) */
    return quick_two_sum(y, (0.5f * y) * e);
}

#endif  /* ORACLE_DF32_OPS_H_ */
