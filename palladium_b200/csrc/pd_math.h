// pd_math.h -- arithmetic building blocks shared by every kernel family.
//
// Everything here compiles both as CUDA device code (nvcc, sm_100a) and as
// plain C++ on the host, and produces the same bits on both, because each
// operation is spelled with an explicit rounding (`__fadd_rn`, `__fmul_rn`,
// `__fmaf_rn`, `__fdiv_rn`, `__fsqrt_rn` on the device; the IEEE operators
// and `fmaf` on the host, where the translation unit must be built with
// `-ffp-contract=off`).  No compiler flag (`-fmad`, `-use_fast_math`) can
// contract, reassociate or approximate what is written through these helpers.
//
// Contents
//   * Threefry-2x32-20 counter RNG, `random_bits`, `fold_in` and the
//     bits -> uniform[0,1) transform, as specified by the reference emitter
//     (src/palladium/emit/rules.py:121-201; op chain of `uniform` named at
//     tests/test_10_random_bits.py:3-7).
//   * df32 ("double-float") compensated arithmetic: error-free transforms and
//     add / sub / mul / div / sqrt on (hi, lo) float pairs.  The reference
//     calls an external prelude for add/sub/mul (examples/05_df32_precision.py:
//     28-30); these are the textbook algorithms (Knuth TwoSum, Dekker
//     FastTwoSum, FMA TwoProd).
//   * pd_powf: a deterministic single-precision pow built only from the
//     helpers above plus integer bit operations, used by the SAFE build of the
//     adaptive integrator so that accept/reject decisions are reproducible
//     bit for bit on any IEEE machine.
#ifndef PD_MATH_H_
#define PD_MATH_H_

#if defined(__CUDACC_RTC__)
// Run-time compilation has no host headers; the device math functions are built in.
typedef unsigned int uint32_t;
typedef int int32_t;
typedef unsigned long long uint64_t;
typedef long long int64_t;
#else
#include <stdint.h>
#include <math.h>
#include <string.h>
#endif

#if defined(__CUDACC__)
#define PD_HD __host__ __device__ __forceinline__
#else
#define PD_HD static inline
#endif

// ---------------------------------------------------------------------------
// Rounding-explicit scalar operations.
// ---------------------------------------------------------------------------
#if defined(__CUDA_ARCH__)
PD_HD float pd_add(float a, float b) { return __fadd_rn(a, b); }
PD_HD float pd_sub(float a, float b) { return __fsub_rn(a, b); }
PD_HD float pd_mul(float a, float b) { return __fmul_rn(a, b); }
PD_HD float pd_fma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
PD_HD float pd_div(float a, float b) { return __fdiv_rn(a, b); }
PD_HD float pd_sqrt(float a) { return __fsqrt_rn(a); }
PD_HD uint32_t pd_f2u(float f) { return __float_as_uint(f); }
PD_HD float pd_u2f(uint32_t u) { return __uint_as_float(u); }
#else
PD_HD float pd_add(float a, float b) { return a + b; }
PD_HD float pd_sub(float a, float b) { return a - b; }
PD_HD float pd_mul(float a, float b) { return a * b; }
PD_HD float pd_fma(float a, float b, float c) { return fmaf(a, b, c); }
PD_HD float pd_div(float a, float b) { return a / b; }
PD_HD float pd_sqrt(float a) { return sqrtf(a); }
PD_HD uint32_t pd_f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
PD_HD float pd_u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
#endif

// a / b, correctly rounded (the value IEEE division returns), for a non-negative
// numerator and a positive denominator -- the quotients of an error norm,
// |err| / (atol + rtol |y|).  On the device the compiler's IEEE division tests its
// operands and sends many ordinary pairs through a long, data-dependent slow path,
// which also splits the warp; this form has no such path for operands in a stated
// range: b in [2^-60, 2^20) and a zero or in [2^-104, 2^60), for which the quotient
// is zero or normal (2^-124 at the least).  It is the classical
// sequence with fused multiply-adds -- hardware reciprocal, one Newton step, quotient,
// and two residual corrections, each residual a - b q exact -- run on a numerator
// scaled by 2^64 when it is small, so that no intermediate leaves the normal range
// (the scaling is by a power of two, hence exact, and so is scaling the quotient
// back, which stays normal).  Outside the range the IEEE division is used.
// On the host it IS the IEEE division.  tests/test_gpu_edge_cases.py compares the
// two on the device over billions of operand pairs.
#if defined(__CUDA_ARCH__)
PD_HD float pd_div_nonneg(float a, float b) {
    const uint32_t ia = __float_as_uint(a), ib = __float_as_uint(b);
    const bool b_ok = (ib - 0x21800000u) < 0x28000000u;                       // 2^-60 <= b < 2^20 (positive, finite)
    const bool a_ok = ia == 0u || (ia - 0x0B800000u) < 0x52000000u;           // +0, or 2^-104 <= a < 2^60
    if (!(a_ok && b_ok)) return __fdiv_rn(a, b);
    const bool small = ia < 0x21800000u;                                      // a < 2^-60: work on a 2^64
    const float as = small ? __fmul_rn(a, 18446744073709551616.0f) : a;
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(b));
    y = __fmaf_rn(y, __fmaf_rn(-b, y, 1.0f), y);
    float q = __fmul_rn(as, y);
    q = __fmaf_rn(__fmaf_rn(-b, q, as), y, q);
    q = __fmaf_rn(__fmaf_rn(-b, q, as), y, q);
    return small ? __fmul_rn(q, 5.42101086242752217e-20f) : q;
}
// Two such quotients at once: the Newton and residual steps, all fused multiply-adds, on packed
// f32x2 instructions (each half rounds as the scalar sequence does); operands outside the fast
// range send both quotients down the scalar function.
PD_HD void pd_div_nonneg_pair(float a1, float b1, float a2, float b2, float* q1, float* q2) {
    const uint32_t ia1 = __float_as_uint(a1), ib1 = __float_as_uint(b1);
    const uint32_t ia2 = __float_as_uint(a2), ib2 = __float_as_uint(b2);
    const bool ok = (ib1 - 0x21800000u) < 0x28000000u && (ib2 - 0x21800000u) < 0x28000000u &&
                    (ia1 == 0u || (ia1 - 0x0B800000u) < 0x52000000u) &&
                    (ia2 == 0u || (ia2 - 0x0B800000u) < 0x52000000u);
    if (!ok) {
        *q1 = pd_div_nonneg(a1, b1);
        *q2 = pd_div_nonneg(a2, b2);
        return;
    }
    const bool small1 = ia1 < 0x21800000u, small2 = ia2 < 0x21800000u;
    const float2 as = make_float2(small1 ? __fmul_rn(a1, 18446744073709551616.0f) : a1,
                                  small2 ? __fmul_rn(a2, 18446744073709551616.0f) : a2);
    const float2 nb = make_float2(-b1, -b2), one = make_float2(1.0f, 1.0f);
    float y1, y2;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y1) : "f"(b1));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y2) : "f"(b2));
    float2 y = make_float2(y1, y2);
    y = __ffma2_rn(y, __ffma2_rn(nb, y, one), y);
    float2 q = __fmul2_rn(as, y);          // consumed by fused multiply-adds only
    q = __ffma2_rn(__ffma2_rn(nb, q, as), y, q);
    q = __ffma2_rn(__ffma2_rn(nb, q, as), y, q);
    *q1 = small1 ? __fmul_rn(q.x, 5.42101086242752217e-20f) : q.x;
    *q2 = small2 ? __fmul_rn(q.y, 5.42101086242752217e-20f) : q.y;
}
#else
PD_HD float pd_div_nonneg(float a, float b) { return a / b; }
PD_HD void pd_div_nonneg_pair(float a1, float b1, float a2, float b2, float* q1, float* q2) {
    *q1 = a1 / b1;
    *q2 = a2 / b2;
}
#endif

// NaN-propagating min / max: the semantics of the staged `max` / `min`
// primitives the reference kernels use (jnp.maximum / jnp.minimum).
// On the device they are single instructions (max.NaN / min.NaN): a NaN operand gives the canonical
// NaN where the host form hands on the operand's own NaN, which no comparison of values can tell
// apart; for a +0 / -0 pair the instruction orders -0 below +0 and the host form returns its second
// operand, a case the callers never produce (they compare non-negative quantities).
#if defined(__CUDA_ARCH__)
PD_HD float pd_max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
PD_HD float pd_min_nan(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
#else
PD_HD float pd_max_nan(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    return a > b ? a : b;
}
PD_HD float pd_min_nan(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    return a < b ? a : b;
}
#endif

// ---------------------------------------------------------------------------
// Threefry-2x32-20.
// ---------------------------------------------------------------------------
PD_HD uint32_t pd_rotl32(uint32_t v, int r) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_l(v, v, r);
#else
    return (v << r) | (v >> (32 - r));
#endif
}

typedef struct pd_u32x2 { uint32_t a, b; } pd_u32x2;

// One Threefry-2x32-20 block: key (k0, k1), counter words (c0, c1).
// Five groups of four mix rounds; rotation sets alternate between
// {13,15,26,6} and {17,29,16,24}; after group g (1-based) the key schedule
// adds ks[g % 3] to the first word and ks[(g+1) % 3] + g to the second.
PD_HD pd_u32x2 pd_threefry2x32(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1) {
    const uint32_t ks0 = k0, ks1 = k1, ks2 = k0 ^ k1 ^ 0x1BD11BDAu;
    uint32_t x0 = c0 + ks0;
    uint32_t x1 = c1 + ks1;
#define PD_TF_MIX(R) { x0 += x1; x1 = pd_rotl32(x1, (R)); x1 ^= x0; }
    PD_TF_MIX(13) PD_TF_MIX(15) PD_TF_MIX(26) PD_TF_MIX(6)
    x0 += ks1; x1 += ks2 + 1u;
    PD_TF_MIX(17) PD_TF_MIX(29) PD_TF_MIX(16) PD_TF_MIX(24)
    x0 += ks2; x1 += ks0 + 2u;
    PD_TF_MIX(13) PD_TF_MIX(15) PD_TF_MIX(26) PD_TF_MIX(6)
    x0 += ks0; x1 += ks1 + 3u;
    PD_TF_MIX(17) PD_TF_MIX(29) PD_TF_MIX(16) PD_TF_MIX(24)
    x0 += ks1; x1 += ks2 + 4u;
    PD_TF_MIX(13) PD_TF_MIX(15) PD_TF_MIX(26) PD_TF_MIX(6)
    x0 += ks2; x1 += ks0 + 5u;
#undef PD_TF_MIX
    pd_u32x2 out; out.a = x0; out.b = x1;
    return out;
}

// random_bits(key, shape)[flat]: counter = (0, flat index); the two output
// words are folded with xor into one 32-bit draw.
PD_HD uint32_t pd_random_bits(uint32_t k0, uint32_t k1, uint32_t flat_index) {
    pd_u32x2 r = pd_threefry2x32(k0, k1, 0u, flat_index);
    return r.a ^ r.b;
}

// fold_in(key, data): counter = (0, data); both output words form the new key.
PD_HD pd_u32x2 pd_fold_in(uint32_t k0, uint32_t k1, uint32_t data) {
    return pd_threefry2x32(k0, k1, 0u, data);
}

// uniform [0, 1): keep the top 23 bits as a mantissa under exponent 0
// (a float in [1, 2)), then subtract one.
PD_HD float pd_bits_to_uniform(uint32_t bits) {
    return pd_sub(pd_u2f((bits >> 9) | 0x3F800000u), 1.0f);
}

// ---------------------------------------------------------------------------
// pcg_hash counter RNG of the reference's hand-written GBM kernel
// (examples/03_sde_montecarlo.py:38-49): one multiply-add, a data-dependent
// shift-xor, one multiply, one shift-xor; the uniform is (hash + 0.5) * 2^-32,
// an open-interval value that is safe under log().
// ---------------------------------------------------------------------------
PD_HD uint32_t pd_pcg_hash(uint32_t v) {
    const uint32_t state = v * 747796405u + 2891336453u;
    const uint32_t word = ((state >> ((state >> 28) + 4u)) ^ state) * 277803737u;
    return (word >> 22) ^ word;
}
PD_HD float pd_pcg_uniform01(uint32_t v) {
#if defined(__CUDA_ARCH__)
    const float h = __uint2float_rn(pd_pcg_hash(v));
#else
    const float h = (float)pd_pcg_hash(v);
#endif
    return pd_mul(pd_add(h, 0.5f), 2.3283064365386963e-10f);  // 2^-32
}

// ---------------------------------------------------------------------------
// df32: value = hi + lo with |lo| <= ulp(hi)/2.
// ---------------------------------------------------------------------------
typedef struct pd_df32 { float hi, lo; } pd_df32;

PD_HD pd_df32 pd_df_make(float hi, float lo) { pd_df32 r; r.hi = hi; r.lo = lo; return r; }
PD_HD pd_df32 pd_df_from_float(float a) { return pd_df_make(a, 0.0f); }
PD_HD float pd_df_to_float(pd_df32 a) { return pd_add(a.hi, a.lo); }

// Knuth TwoSum: s + e == a + b exactly, no ordering assumption (6 flops).
PD_HD pd_df32 pd_two_sum(float a, float b) {
    float s = pd_add(a, b);
    float bb = pd_sub(s, a);
    float e = pd_add(pd_sub(a, pd_sub(s, bb)), pd_sub(b, bb));
    return pd_df_make(s, e);
}
// Dekker FastTwoSum: exact when |a| >= |b| (3 flops).
PD_HD pd_df32 pd_fast_two_sum(float a, float b) {
    float s = pd_add(a, b);
    float e = pd_sub(b, pd_sub(s, a));
    return pd_df_make(s, e);
}
// TwoProd with FMA: p + e == a * b exactly (2 flops).
PD_HD pd_df32 pd_two_prod(float a, float b) {
    float p = pd_mul(a, b);
    float e = pd_fma(a, b, -p);
    return pd_df_make(p, e);
}

// Accurate df32 addition (both low-order words go through a TwoSum).
PD_HD pd_df32 pd_df_add(pd_df32 a, pd_df32 b) {
    pd_df32 s = pd_two_sum(a.hi, b.hi);
    pd_df32 t = pd_two_sum(a.lo, b.lo);
    s.lo = pd_add(s.lo, t.hi);
    s = pd_fast_two_sum(s.hi, s.lo);
    s.lo = pd_add(s.lo, t.lo);
    return pd_fast_two_sum(s.hi, s.lo);
}
PD_HD pd_df32 pd_df_neg(pd_df32 a) { return pd_df_make(-a.hi, -a.lo); }
PD_HD pd_df32 pd_df_sub(pd_df32 a, pd_df32 b) { return pd_df_add(a, pd_df_neg(b)); }

PD_HD pd_df32 pd_df_mul(pd_df32 a, pd_df32 b) {
    pd_df32 p = pd_two_prod(a.hi, b.hi);
    p.lo = pd_fma(a.hi, b.lo, p.lo);
    p.lo = pd_fma(a.lo, b.hi, p.lo);
    return pd_fast_two_sum(p.hi, p.lo);
}

// df32 / df32: two quotient digits from IEEE float division, each followed by
// an exact residual update, plus a third correction digit.
PD_HD pd_df32 pd_df_div(pd_df32 a, pd_df32 b) {
    float q1 = pd_div(a.hi, b.hi);
    pd_df32 r = pd_df_sub(a, pd_df_mul(pd_df_from_float(q1), b));
    float q2 = pd_div(r.hi, b.hi);
    r = pd_df_sub(r, pd_df_mul(pd_df_from_float(q2), b));
    float q3 = pd_div(r.hi, b.hi);
    pd_df32 q = pd_fast_two_sum(q1, q2);
    return pd_df_add(q, pd_df_from_float(q3));
}

// 1 / b: one IEEE quotient digit q = 1 / b.hi, then one Newton step carried out
// with error-free products: e = 1 - b q is formed exactly (b.hi q as a TwoProd,
// 1 - p.hi exact by Sterbenz), and 1 / b = q (1 + e + O(e^2)), e ~ 2^-24.
PD_HD pd_df32 pd_df_recip(pd_df32 b) {
    const float q = pd_div(1.0f, b.hi);
    pd_df32 p = pd_two_prod(b.hi, q);
    p.lo = pd_fma(b.lo, q, p.lo);
    const float e = pd_sub(pd_sub(1.0f, p.hi), p.lo);
    return pd_fast_two_sum(q, pd_mul(q, e));
}

// 2 a, exact.
PD_HD pd_df32 pd_df_twice(pd_df32 a) { return pd_df_make(pd_add(a.hi, a.hi), pd_add(a.lo, a.lo)); }

// sqrt(df32): IEEE float sqrt as the seed, one Newton correction carried out
// in df32:  r = s + (a - s*s) / (2 s).   a must be >= 0; sqrt(0) = 0.
PD_HD pd_df32 pd_df_sqrt(pd_df32 a) {
    float s = pd_sqrt(a.hi);
    if (s == 0.0f) return pd_df_make(0.0f, 0.0f);
    pd_df32 ss = pd_two_prod(s, s);
    pd_df32 d = pd_df_sub(a, ss);
    float corr = pd_div(d.hi, pd_add(s, s));
    return pd_fast_two_sum(s, corr);
}

// 1 / sqrt(a) for a > 0.  The seed is the integer estimate 0x5F375A86 - (bits >> 1)
// (within 3.5 %), refined by three float Newton steps y <- y (3/2 - (a/2) y^2) to
// float accuracy; every operation is a plain IEEE one, so host and device agree bit
// for bit (the hardware's approximate rsqrt would be shorter but is not reproducible
// off the GPU).  The last correction is carried out in df32 and to second order,
// rs = y (1 + e/2 + 3 e^2/8) with e = 1 - a y^2 formed from error-free products
// (e ~ 2^-22, so what is left is O(e^3), far below the pair's 2^-48).
PD_HD pd_df32 pd_df_rsqrt(pd_df32 a) {
    const float half_a = pd_mul(0.5f, a.hi);
    float y = pd_u2f(0x5F375A86u - (pd_f2u(a.hi) >> 1));
    y = pd_mul(y, pd_sub(1.5f, pd_mul(half_a, pd_mul(y, y))));
    y = pd_mul(y, pd_sub(1.5f, pd_mul(half_a, pd_mul(y, y))));
    y = pd_mul(y, pd_sub(1.5f, pd_mul(half_a, pd_mul(y, y))));
    const pd_df32 t = pd_df_mul(a, pd_two_prod(y, y));           // a y^2 = 1 + O(2^-22)
    float e = pd_sub(pd_sub(1.0f, t.hi), t.lo);                  // 1 - t.hi is exact (Sterbenz)
    e = pd_fma(pd_mul(0.75f, e), e, e);                          // e + 3 e^2 / 4
    return pd_fast_two_sum(y, pd_mul(pd_mul(0.5f, y), e));
}

// ---------------------------------------------------------------------------
// pd_powf: deterministic x**y for x >= 0.
//   log2(x) is formed in df32 from x = 2^e * m, m in [sqrt(1/2), sqrt(2)],
//   s = (m-1)/(m+1), log(m) = 2 s + 2 s^3/3 + ... ; the product y * log2(x)
//   is split into an integer n and a fraction f, |f| <= 1/2, and 2^f is a
//   degree-7 polynomial.  Measured against double-precision pow rounded to
//   float the result is within 1 ulp over the tested domain.
//   Domain rules: NaN in -> NaN; x < 0 -> NaN; y == 0 -> 1; x == 0 -> 0 (y>0)
//   or +inf (y<0); x == +inf -> +inf (y>0) or 0 (y<0).
// ---------------------------------------------------------------------------
PD_HD float pd_exp2_scale(float r, int n) {
    // r * 2^n for r in [1/2, 2] and n in [-160, 254].  Every multiply but the
    // last is exact, so a subnormal result is rounded exactly once.
    if (n > 127) {
        r = pd_mul(r, pd_u2f(254u << 23));       // * 2^127
        n -= 127;
        if (n > 127) n = 127;
    }
    if (n < -126) {
        if (n < -160) n = -160;
        r = pd_mul(r, pd_u2f((uint32_t)(n + 64 + 127) << 23));  // * 2^(n+64), normal
        n = -64;
    }
    return pd_mul(r, pd_u2f((uint32_t)(n + 127) << 23));
}

// log2(x) as a df32 value, for finite x > 0 (subnormals included).
PD_HD pd_df32 pd_log2_df(float x) {
    uint32_t ix = pd_f2u(x);
    int e = 0;
    if (ix < 0x00800000u) {  // subnormal: scale up by 2^24 (exact)
        ix = pd_f2u(pd_mul(x, 16777216.0f));
        e = -24;
    }
    e += (int)(ix >> 23) - 127;
    float m = pd_u2f((ix & 0x007FFFFFu) | 0x3F800000u);  // [1, 2)
    if (m > 1.41421354f) { m = pd_mul(m, 0.5f); e += 1; }

    // s = (m - 1) / (m + 1) as a df32 value.
    float num = pd_sub(m, 1.0f);                 // exact
    pd_df32 den = pd_two_sum(m, 1.0f);
    float s_hi = pd_div(num, den.hi);
    float res = pd_fma(-s_hi, den.hi, num);      // exact residual
    res = pd_fma(-s_hi, den.lo, res);
    float s_lo = pd_div(res, den.hi);

    // log(m) = 2 s + s * q(z), z = s^2.
    float z = pd_mul(s_hi, s_hi);
    float q = 0.153846154f;                      // 2/13
    q = pd_fma(q, z, 0.181818182f);              // 2/11
    q = pd_fma(q, z, 0.222222222f);              // 2/9
    q = pd_fma(q, z, 0.285714286f);              // 2/7
    q = pd_fma(q, z, 0.4f);                      // 2/5
    q = pd_fma(q, z, 0.666666667f);              // 2/3
    q = pd_mul(q, z);
    float tail = pd_fma(s_hi, q, pd_add(s_lo, s_lo));
    pd_df32 L = pd_fast_two_sum(pd_add(s_hi, s_hi), tail);

    // log2(m) = L * log2(e), log2(e) = 1.44269502162933349609375 + 1.925963033500011e-8
    const float c_hi = 1.44269502f, c_lo = 1.92596303e-8f;
    pd_df32 P = pd_two_prod(L.hi, c_hi);
    P.lo = pd_fma(L.hi, c_lo, P.lo);
    P.lo = pd_fma(L.lo, c_hi, P.lo);

    // T = e + P
    pd_df32 T = pd_two_sum((float)e, P.hi);
    T.lo = pd_add(T.lo, P.lo);
    return pd_fast_two_sum(T.hi, T.lo);
}

// 2^(y * T) for a df32 exponent factor T = log2(x): the second half of pd_powf.
PD_HD float pd_exp2_of_product(float y, pd_df32 T) {
    const float inf = pd_u2f(0x7F800000u);
    pd_df32 W = pd_two_prod(y, T.hi);
    W.lo = pd_fma(y, T.lo, W.lo);

    if (!(W.hi < 129.0f)) return inf;
    if (!(W.hi > -151.0f)) return 0.0f;

    float nf = floorf(pd_add(W.hi, 0.5f));
    float f = pd_add(pd_sub(W.hi, nf), W.lo);
    int n = (int)nf;

    // 2^f - 1 = f * (ln2 + f * (ln2^2/2 + ...)), Taylor coefficients ln2^k / k!
    float p = 1.52527338e-5f;                    // ln2^7/7!
    p = pd_fma(p, f, 1.54035304e-4f);            // ln2^6/6!
    p = pd_fma(p, f, 1.33335581e-3f);            // ln2^5/5!
    p = pd_fma(p, f, 9.61812911e-3f);            // ln2^4/4!
    p = pd_fma(p, f, 5.55041087e-2f);            // ln2^3/3!
    p = pd_fma(p, f, 2.40226507e-1f);            // ln2^2/2!
    p = pd_fma(p, f, 6.93147181e-1f);            // ln2
    float r = pd_fma(p, f, 1.0f);
    return pd_exp2_scale(r, n);
}

// 1 when (x, y) needs one of pd_powf's domain rules instead of the log/exp path.
PD_HD int pd_pow_is_special(float x, float y) {
    const float inf = pd_u2f(0x7F800000u);
    return (x != x) || (y != y) || y == 0.0f || !(x > 0.0f) || x == inf || y == inf || y == -inf;
}

PD_HD float pd_powf(float x, float y) {
    if (x != x || y != y) return x + y;
    if (y == 0.0f) return 1.0f;
    if (x < 0.0f) return pd_u2f(0x7FC00000u);
    const float inf = pd_u2f(0x7F800000u);
    if (x == 0.0f) return y > 0.0f ? 0.0f : inf;
    if (x == inf) return y > 0.0f ? inf : 0.0f;
    if (y == inf) return x > 1.0f ? inf : (x == 1.0f ? 1.0f : 0.0f);
    if (y == -inf) return x > 1.0f ? 0.0f : (x == 1.0f ? 1.0f : inf);
    return pd_exp2_of_product(y, pd_log2_df(x));
}

// x**y1 and x**y2 with one logarithm: bit-identical to two pd_powf calls.
PD_HD void pd_powf_pair(float x, float y1, float y2, float* r1, float* r2) {
    if (pd_pow_is_special(x, y1) || pd_pow_is_special(x, y2)) {
        *r1 = pd_powf(x, y1);
        *r2 = pd_powf(x, y2);
        return;
    }
    const pd_df32 T = pd_log2_df(x);
    *r1 = pd_exp2_of_product(y1, T);
    *r2 = pd_exp2_of_product(y2, T);
}

// ---------------------------------------------------------------------------
// Controller-grade powers.  An adaptive step controller needs (1 / err)**c for
// two small exponents c per attempt, and only to size the next step: accepted
// states are governed by the error norm, not by these powers.  pd_ctrl_powers
// evaluates them as 2**(-c log2(err)) in float arithmetic alone -- one shared
// logarithm (exponent + a degree-9 polynomial in m - 1, m in [sqrt(1/2), sqrt(2)])
// and a degree-6 polynomial for 2**f, |f| <= 1/2 -- without forming 1 / err at
// all: about 60 operations for the pair, against about 150 for two pd_powf
// calls plus a division.  Measured against double precision over err in
// [1e-9, 1e9] the result is within 7 ulp (mean 1.3 ulp); the error is that of
// rounding log2(err), up to 30 in magnitude, to float.  Every operation is an
// explicitly rounded one, so host and device agree bit for bit, which is what
// pins integer step counts.  Arguments outside the normal positive range (zero,
// subnormal, negative, infinite, NaN) and products outside [-120, 120] take
// 1 / err and pd_powf, with pd_powf's domain rules.
// ---------------------------------------------------------------------------
PD_HD float pd_ctrl_log2(float x) {   // x: positive, normal, finite
    const uint32_t ix = pd_f2u(x);
    int e = (int)(ix >> 23) - 127;
    float m = pd_u2f((ix & 0x007FFFFFu) | 0x3F800000u);  // [1, 2)
    if (m > 1.41421354f) { m = pd_mul(m, 0.5f); e += 1; }
    const float t = pd_sub(m, 1.0f);                      // exact
    float q = -1.129741669e-01f;
    q = pd_fma(q, t, 1.878263354e-01f);
    q = pd_fma(q, t, -1.906127632e-01f);
    q = pd_fma(q, t, 2.042960823e-01f);
    q = pd_fma(q, t, -2.396365702e-01f);
    q = pd_fma(q, t, 2.885852754e-01f);
    q = pd_fma(q, t, -3.606964350e-01f);
    q = pd_fma(q, t, 4.808979034e-01f);
    q = pd_fma(q, t, -7.213473320e-01f);
    q = pd_fma(q, t, 1.442695022e+00f);
    return pd_fma(t, q, (float)e);
}

#define PD_EXP2_C6 1.546973217e-04f
#define PD_EXP2_C5 1.339086681e-03f
#define PD_EXP2_C4 9.618030861e-03f
#define PD_EXP2_C3 5.550356954e-02f
#define PD_EXP2_C2 2.402265072e-01f
#define PD_EXP2_C1 6.931471825e-01f
PD_HD float pd_ctrl_exp2(float w) {   // |w| <= 120
    const float nf = floorf(pd_add(w, 0.5f));
    const float f = pd_sub(w, nf);                        // exact, |f| <= 1/2
    float p = PD_EXP2_C6;
    p = pd_fma(p, f, PD_EXP2_C5);
    p = pd_fma(p, f, PD_EXP2_C4);
    p = pd_fma(p, f, PD_EXP2_C3);
    p = pd_fma(p, f, PD_EXP2_C2);
    p = pd_fma(p, f, PD_EXP2_C1);
    const float r = pd_fma(p, f, 1.0f);                   // 2**0 is exactly 1
    return pd_mul(r, pd_u2f((uint32_t)((int)nf + 127) << 23));
}

// r1 = (1 / err)**c1, r2 = (1 / err)**c2.
PD_HD void pd_ctrl_powers(float err, float c1, float c2, float* r1, float* r2) {
    const uint32_t ix = pd_f2u(err);
    if (ix - 0x00800000u < 0x7F000000u) {                 // positive, normal, finite
        const float l = -pd_ctrl_log2(err);               // log2(1 / err)
        const float w1 = pd_mul(c1, l), w2 = pd_mul(c2, l);
        if (fabsf(w1) <= 120.0f && fabsf(w2) <= 120.0f) {
#if defined(__CUDA_ARCH__)
            // pd_ctrl_exp2 for both arguments at once on packed f32x2 instructions: each half goes
            // through the operations of the scalar function with the same roundings (w - nf as the
            // exact fma nf * (-1) + w; no packed multiply here has an add as its only consumer, which
            // is the one pattern the assembler would fuse).
            const float2 w = make_float2(w1, w2);
            const float2 nf = make_float2(floorf(pd_add(w1, 0.5f)), floorf(pd_add(w2, 0.5f)));
            const float2 f = __ffma2_rn(nf, make_float2(-1.0f, -1.0f), w);
            float2 q = make_float2(PD_EXP2_C6, PD_EXP2_C6);
            q = __ffma2_rn(q, f, make_float2(PD_EXP2_C5, PD_EXP2_C5));
            q = __ffma2_rn(q, f, make_float2(PD_EXP2_C4, PD_EXP2_C4));
            q = __ffma2_rn(q, f, make_float2(PD_EXP2_C3, PD_EXP2_C3));
            q = __ffma2_rn(q, f, make_float2(PD_EXP2_C2, PD_EXP2_C2));
            q = __ffma2_rn(q, f, make_float2(PD_EXP2_C1, PD_EXP2_C1));
            q = __ffma2_rn(q, f, make_float2(1.0f, 1.0f));
            const float2 scale = make_float2(pd_u2f((uint32_t)((int)nf.x + 127) << 23),
                                             pd_u2f((uint32_t)((int)nf.y + 127) << 23));
            const float2 r = __fmul2_rn(q, scale);
            *r1 = r.x;
            *r2 = r.y;
#else
            *r1 = pd_ctrl_exp2(w1);
            *r2 = pd_ctrl_exp2(w2);
#endif
            return;
        }
    }
    const float inv = pd_div(1.0f, err);
    *r1 = pd_powf(inv, c1);
    *r2 = pd_powf(inv, c2);
}

// ---------------------------------------------------------------------------
// Embedded explicit Runge-Kutta pairs of order 5(4) with seven stages, the last of which is the
// slope at the new point (first-same-as-last).  Row s of A (s = 1..6) holds the s coefficients of
// stage s + 1; row 6 is the fifth-order weight vector.  E holds the weights of the error estimate,
// err = h * sum_j E[j] k_j (fifth-order minus fourth-order solution).  Every coefficient is the
// float nearest to the double expression written here, on the GPU and in the CPU oracle alike.
//   Dormand and Prince (1980), "A family of embedded Runge-Kutta formulae", J. Comp. Appl. Math. 6.
//   Tsitouras (2011), "Runge-Kutta pairs of order 5(4) satisfying only the first column
//   simplifying assumption", Comput. Math. Appl. 62 -- the pair the reference's CPU comparison
//   runs (benchmarks/bench_ensembles.py: diffrax.Tsit5).
// ---------------------------------------------------------------------------
#define PD_ERK_STAGES 7
#define PD_RKF(x) ((float)(x))

#define PD_DOPRI5_C {PD_RKF(0.0), PD_RKF(1.0 / 5.0), PD_RKF(3.0 / 10.0), PD_RKF(4.0 / 5.0), PD_RKF(8.0 / 9.0), \
                     PD_RKF(1.0), PD_RKF(1.0)}
#define PD_DOPRI5_A {                                                                                            \
    {PD_RKF(1.0 / 5.0), 0, 0, 0, 0, 0},                                                                          \
    {PD_RKF(3.0 / 40.0), PD_RKF(9.0 / 40.0), 0, 0, 0, 0},                                                        \
    {PD_RKF(44.0 / 45.0), PD_RKF(-56.0 / 15.0), PD_RKF(32.0 / 9.0), 0, 0, 0},                                    \
    {PD_RKF(19372.0 / 6561.0), PD_RKF(-25360.0 / 2187.0), PD_RKF(64448.0 / 6561.0), PD_RKF(-212.0 / 729.0), 0, 0}, \
    {PD_RKF(9017.0 / 3168.0), PD_RKF(-355.0 / 33.0), PD_RKF(46732.0 / 5247.0), PD_RKF(49.0 / 176.0),             \
     PD_RKF(-5103.0 / 18656.0), 0},                                                                              \
    {PD_RKF(35.0 / 384.0), 0, PD_RKF(500.0 / 1113.0), PD_RKF(125.0 / 192.0), PD_RKF(-2187.0 / 6784.0),           \
     PD_RKF(11.0 / 84.0)}}
#define PD_DOPRI5_E {PD_RKF(71.0 / 57600.0), 0, PD_RKF(-71.0 / 16695.0), PD_RKF(71.0 / 1920.0),                  \
                     PD_RKF(-17253.0 / 339200.0), PD_RKF(22.0 / 525.0), PD_RKF(-1.0 / 40.0)}

#define PD_TSIT5_C {PD_RKF(0.0), PD_RKF(0.161), PD_RKF(0.327), PD_RKF(0.9), PD_RKF(0.9800255409045097),          \
                    PD_RKF(1.0), PD_RKF(1.0)}
#define PD_TSIT5_A {                                                                                             \
    {PD_RKF(0.161), 0, 0, 0, 0, 0},                                                                              \
    {PD_RKF(-0.008480655492356989), PD_RKF(0.335480655492357), 0, 0, 0, 0},                                      \
    {PD_RKF(2.8971530571054935), PD_RKF(-6.359448489975075), PD_RKF(4.3622954328695815), 0, 0, 0},               \
    {PD_RKF(5.325864828439257), PD_RKF(-11.748883564062828), PD_RKF(7.4955393428898365),                         \
     PD_RKF(-0.09249506636175525), 0, 0},                                                                        \
    {PD_RKF(5.86145544294642), PD_RKF(-12.92096931784711), PD_RKF(8.159367898576159),                            \
     PD_RKF(-0.071584973281401), PD_RKF(-0.028269050394068383), 0},                                              \
    {PD_RKF(0.09646076681806523), PD_RKF(0.01), PD_RKF(0.4798896504144996), PD_RKF(1.379008574103742),           \
     PD_RKF(-3.290069515436081), PD_RKF(2.324710524099774)}}
#define PD_TSIT5_E {PD_RKF(-0.00178001105222577714), PD_RKF(-0.0008164344596567469),                             \
                    PD_RKF(0.007880878010261995), PD_RKF(-0.1447110071732629), PD_RKF(0.5823571654525552),       \
                    PD_RKF(-0.45808210592918697), PD_RKF(1.0 / 66.0)}

#endif  // PD_MATH_H_
