/* oracle.c -- CPU restatement of the reference's ensemble-integrator kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import, link
 * or execute this file; it is the checker the CUDA kernels are compared with
 * (tests/, the smoke check, and the CPU-baseline leg of the benchmark).
 *
 * The reference's own oracle is `pl.pallas_call(..., interpret=True)`
 * (src/palladium/__init__.py:110), which needs JAX and cannot run where this
 * is built.  Each function below restates one reference kernel operation by
 * operation, in the order the kernel body stages them, in IEEE binary32 with
 * no contraction (build with -ffp-contract=off, never -ffast-math).  Python
 * float constants are folded in double first and rounded to float once, as
 * JAX's weak typing does (visible in the literals of
 * tests/golden/rk4_lotka_volterra.metal:90,186,254).
 *
 * Pinning status
 *   rk4 lotka-volterra : pinned -- bit-identical to the reference's emitted
 *                        kernel tests/golden/rk4_lotka_volterra.metal compiled
 *                        as C++ (oracle/build.py builds it into oracle/_ref/).
 *   threefry block, random_bits, fold_in : pinned -- bit-identical to the
 *                        statements the reference's emitter writes
 *                        (`_emit_threefry2x32`, src/palladium/emit/rules.py:121-165,
 *                        run where it lies and compiled as C by oracle/build.py
 *                        into oracle/_ref/), with the counters of the random_bits
 *                        and fold_in rules (:168-201).
 *   uniform            : PARITY UNPINNED -- the reference checks it against a
 *                        live jax.random and stores no vectors
 *                        (tests/test_10_random_bits.py:42-54); the op chain is
 *                        the one named at tests/test_10_random_bits.py:3-7.
 *   float64 RK4 truth  : pinned -- bit-identical to the reference's NumPy
 *                        `float64_reference` (examples/05_df32_precision.py:95-109).
 *   GBM with pcg_hash  : pinned -- bit-identical to the reference's hand-written
 *                        MSL kernel (GBM_MSL, examples/03_sde_montecarlo.py:34-70)
 *                        compiled as C++ through oracle/msl_shim.
 *   adaptive BS3(2), GBM with Threefry, Gray-Scott : pinned -- bit-identical to
 *                        the reference's own kernel functions (examples/02:69-171,
 *                        examples/03:97-119, examples/04:61-74) executed on NumPy
 *                        stand-ins for the jax / pl names they use
 *                        (tests/golden/pallas_numpy.py, tests/golden/make_golden.py),
 *                        with this C library's pow / exp / log / cos.
 *   df32 : kernel structure pinned (bit-identical to the reference's DF32_KERNEL
 *                        text, examples/05_df32_precision.py:27-80, compiled on
 *                        df32_ops.h); arithmetic PARITY UNPINNED -- the prelude
 *                        (df_add/df_sub/df_mul) lives in the external
 *                        metal-runtime project, which is not in the tree;
 *                        textbook error-free transforms are used and checked for
 *                        exactness with rational arithmetic.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* The deterministic pow used by the SAFE build of the adaptive kernel is a
 * product-defined function (the reference has none); the "exact" flavour of
 * the adaptive oracle must use the very same algorithm to be able to compare
 * integer step counts bit for bit, so it is included from the product tree.
 * Everything else in this file is restated independently. */
#include "../palladium_b200/csrc/pd_math.h"

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Threefry-2x32-20 (src/palladium/emit/rules.py:121-165)                      */
/* ------------------------------------------------------------------------- */
static inline uint32_t rotl(uint32_t x, unsigned r) { return (x << r) | (x >> (32u - r)); }

static void threefry(uint32_t k1, uint32_t k2, uint32_t c_hi, uint32_t c_lo, uint32_t* o0, uint32_t* o1) {
    static const unsigned rot[2][4] = {{13, 15, 26, 6}, {17, 29, 16, 24}};
    /* (rotation set, ks index added to x0, ks index added to x1, round counter) */
    static const int sched[5][4] = {{0, 1, 2, 1}, {1, 2, 0, 2}, {0, 0, 1, 3}, {1, 1, 2, 4}, {0, 2, 0, 5}};
    uint32_t ks[3];
    ks[0] = k1; ks[1] = k2; ks[2] = k1 ^ k2 ^ 0x1BD11BDAu;
    uint32_t x0 = c_hi + ks[0];
    uint32_t x1 = c_lo + ks[1];
    for (int g = 0; g < 5; ++g) {
        for (int r = 0; r < 4; ++r) {
            x0 = x0 + x1;
            x1 = rotl(x1, rot[sched[g][0]][r]);
            x1 = x0 ^ x1;
        }
        x0 = x0 + ks[sched[g][1]];
        x1 = x1 + ks[sched[g][2]] + (uint32_t)sched[g][3];
    }
    *o0 = x0; *o1 = x1;
}

/* random_bits: counter (0, flat index), output x0 ^ x1 (rules.py:168-185) */
static uint32_t random_bits_at(uint32_t k1, uint32_t k2, uint32_t idx) {
    uint32_t a, b;
    threefry(k1, k2, 0u, idx, &a, &b);
    return a ^ b;
}
/* uniform: bits >> 9 | 0x3F800000, bitcast, minus 1 (tests/test_10_random_bits.py:3-7) */
static float bits_to_uniform(uint32_t bits) {
    uint32_t u = (bits >> 9) | 0x3F800000u;
    float f;
    memcpy(&f, &u, 4);
    return f - 1.0f;
}

ORC_API void orc_threefry2x32(const uint32_t* key, const uint32_t* ctr, uint32_t* out) {
    threefry(key[0], key[1], ctr[0], ctr[1], &out[0], &out[1]);
}
ORC_API void orc_random_bits(const uint32_t* key, int64_t n, uint32_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = random_bits_at(key[0], key[1], (uint32_t)i);
}
ORC_API void orc_uniform(const uint32_t* key, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = bits_to_uniform(random_bits_at(key[0], key[1], (uint32_t)i));
}
/* fold_in: counter (0, data), new key = (x0, x1) (rules.py:188-201) */
ORC_API void orc_fold_in(const uint32_t* key, const uint32_t* data, int64_t m, uint32_t* out) {
    for (int64_t i = 0; i < m; ++i) threefry(key[0], key[1], 0u, data[i], &out[2 * i], &out[2 * i + 1]);
}
/* per-thread streams: row g = uniform(fold_in(key, g), (count,))
 * (tests/test_10_random_bits.py:78-108) */
ORC_API void orc_fold_uniform(const uint32_t* key, int64_t groups, int64_t count, float* out) {
    for (int64_t g = 0; g < groups; ++g) {
        uint32_t a, b;
        threefry(key[0], key[1], 0u, (uint32_t)g, &a, &b);
        for (int64_t j = 0; j < count; ++j) out[g * count + j] = bits_to_uniform(random_bits_at(a, b, (uint32_t)j));
    }
}

/* ------------------------------------------------------------------------- */
/* Fixed-step RK4 Lotka-Volterra (examples/01_ode_ensembles.py:72-91)          */
/* ------------------------------------------------------------------------- */
ORC_API void orc_lv_rk4(int64_t n, const float* x0, const float* y0, const float* a_, const float* b_,
                        const float* c_, const float* d_, float* xo, float* yo, double dt, int64_t steps) {
    const float hh = (float)(0.5 * dt), hf = (float)dt, h6 = (float)(dt / 6.0);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float a = a_[i], b = b_[i], c = c_[i], d = d_[i];
        float x = x0[i], y = y0[i];
        for (int64_t s = 0; s < steps; ++s) {
            /* rhs(x, y) = (a*x - b*x*y, c*x*y - d*y), left-associated products */
            float k1x = a * x - (b * x) * y, k1y = (c * x) * y - d * y;
            float x2 = x + hh * k1x, y2 = y + hh * k1y;
            float k2x = a * x2 - (b * x2) * y2, k2y = (c * x2) * y2 - d * y2;
            float x3 = x + hh * k2x, y3 = y + hh * k2y;
            float k3x = a * x3 - (b * x3) * y3, k3y = (c * x3) * y3 - d * y3;
            float x4 = x + hf * k3x, y4 = y + hf * k3y;
            float k4x = a * x4 - (b * x4) * y4, k4y = (c * x4) * y4 - d * y4;
            float nx = x + h6 * (((k1x + 2.0f * k2x) + 2.0f * k3x) + k4x);
            float ny = y + h6 * (((k1y + 2.0f * k2y) + 2.0f * k3y) + k4y);
            x = nx; y = ny;
        }
        xo[i] = x; yo[i] = y;
    }
}

/* float64 RK4 of the same system: the truth of examples/05_df32_precision.py:95-109 */
ORC_API void orc_lv_rk4_f64(int64_t n, const float* x0, const float* y0, const float* a_, const float* b_,
                            const float* c_, const float* d_, double* xo, double* yo, double dt, int64_t steps) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const double a = a_[i], b = b_[i], c = c_[i], d = d_[i];
        double x = x0[i], y = y0[i];
        for (int64_t s = 0; s < steps; ++s) {
            double k1x = a * x - b * x * y, k1y = c * x * y - d * y;
            double x2 = x + 0.5 * dt * k1x, y2 = y + 0.5 * dt * k1y;
            double k2x = a * x2 - b * x2 * y2, k2y = c * x2 * y2 - d * y2;
            double x3 = x + 0.5 * dt * k2x, y3 = y + 0.5 * dt * k2y;
            double k3x = a * x3 - b * x3 * y3, k3y = c * x3 * y3 - d * y3;
            double x4 = x + dt * k3x, y4 = y + dt * k3y;
            double k4x = a * x4 - b * x4 * y4, k4y = c * x4 * y4 - d * y4;
            double nx = x + dt / 6.0 * (k1x + 2 * k2x + 2 * k3x + k4x);
            double ny = y + dt / 6.0 * (k1y + 2 * k2y + 2 * k3y + k4y);
            x = nx; y = ny;
        }
        xo[i] = x; yo[i] = y;
    }
}

/* ------------------------------------------------------------------------- */
/* Adaptive Bogacki-Shampine 3(2), FSAL, PI controller, Van der Pol            */
/* (examples/02_adaptive_lockstep.py:69-171).  The loop runs the full          */
/* max_steps trip count, stall iterations included, as the reference does.     */
/* pow_flavour 0: C library powf on 1/err; 1: the deterministic pd_ctrl_powers. */
/* ------------------------------------------------------------------------- */
static inline float max_nan(float a, float b) { return (a != a) ? a : (b != b) ? b : (a > b ? a : b); }
static inline float min_nan(float a, float b) { return (a != a) ? a : (b != b) ? b : (a < b ? a : b); }

ORC_API void orc_vdp_bs32(int64_t n, const float* x0_, const float* v0_, const float* mu_, float* t_out,
                          float* x_out, float* v_out, float* steps_out, float* rejected_out, float* real_out,
                          double t1_, double rtol_, double atol_, double dt0_, double pcoeff, double icoeff,
                          double safety_, double fmin_, double fmax_, int64_t error_order, int64_t max_steps,
                          int pow_flavour) {
    const float T1 = (float)t1_, RTOL = (float)rtol_, ATOL = (float)atol_, DT0 = (float)dt0_;
    const float SAFETY = (float)safety_, FMIN = (float)fmin_, FMAX = (float)fmax_;
    const float coeff1 = (float)((icoeff + pcoeff) / (double)error_order);
    const float coeff2 = (float)(-pcoeff / (double)error_order);
    const float c29 = (float)(2.0 / 9.0), c13 = (float)(1.0 / 3.0), c49 = (float)(4.0 / 9.0);
    const float c724 = (float)(7.0 / 24.0), c14 = (float)(1.0 / 4.0), c18 = (float)(1.0 / 8.0);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < n; ++i) {
        const float mu = mu_[i];
        float t = 0.0f, dt = DT0, x = x0_[i], v = v0_[i];
        float k1x = v, k1v = (mu * (1.0f - x * x)) * v - x;
        float prev_inv_err = 1.0f, prev_err = 1.0f, steps = 0.0f, rejected = 0.0f, real = 0.0f;
        for (int64_t it = 0; it < max_steps; ++it) {
            const int was_real = t < T1;
            dt = min_nan(dt, T1 - t);
            float ax = x + (0.5f * dt) * k1x, av = v + (0.5f * dt) * k1v;
            float k2x = av, k2v = (mu * (1.0f - ax * ax)) * av - ax;
            float bx = x + (0.75f * dt) * k2x, bv = v + (0.75f * dt) * k2v;
            float k3x = bv, k3v = (mu * (1.0f - bx * bx)) * bv - bx;
            float x3 = x + dt * ((c29 * k1x + c13 * k2x) + c49 * k3x);
            float v3 = v + dt * ((c29 * k1v + c13 * k2v) + c49 * k3v);
            float k4x = v3, k4v = (mu * (1.0f - x3 * x3)) * v3 - x3;
            float x2 = x + dt * (((c724 * k1x + c14 * k2x) + c13 * k3x) + c18 * k4x);
            float v2 = v + dt * (((c724 * k1v + c14 * k2v) + c13 * k3v) + c18 * k4v);
            float err_x = x3 - x2, err_v = v3 - v2;
            float err_norm = max_nan(fabsf(err_x) / (ATOL + RTOL * fabsf(x3)),
                                     fabsf(err_v) / (ATOL + RTOL * fabsf(v3)));
            const int accept = err_norm <= 1.0f;
            float t_new = accept ? t + dt : t;
            float x_new = accept ? x3 : x, v_new = accept ? v3 : v;
            float nk1x = accept ? k4x : k1x, nk1v = accept ? k4v : k1v;
            err_norm = max_nan(err_norm, 1e-9f);
            float inv_err = 1.0f / err_norm;
            float pa, pb;
            if (pow_flavour == 1) {
                /* the same two powers, (1/err)**c1 and (1/prev_err)**c2, through the float routine the
                 * CUDA kernel uses (it takes err, not 1/err) */
                float unused;
                pd_ctrl_powers(err_norm, coeff1, coeff1, &pa, &unused);
                pd_ctrl_powers(prev_err, coeff2, coeff2, &pb, &unused);
            } else { pa = powf(inv_err, coeff1); pb = powf(prev_inv_err, coeff2); }
            float factor = (SAFETY * pa) * pb;
            prev_inv_err = accept ? inv_err : prev_inv_err;
            prev_err = accept ? err_norm : prev_err;
            dt = dt * min_nan(max_nan(factor, FMIN), FMAX);
            steps = steps + (accept ? 1.0f : 0.0f);
            rejected = rejected + (accept ? 0.0f : 1.0f);
            real = real + (was_real ? (accept ? 1.0f : 0.0f) : 0.0f);
            t = t_new; x = x_new; v = v_new; k1x = nk1x; k1v = nk1v;
        }
        t_out[i] = t; x_out[i] = x; v_out[i] = v;
        steps_out[i] = steps; rejected_out[i] = rejected; real_out[i] = real;
    }
}

/* ------------------------------------------------------------------------- */
/* GBM Monte Carlo with in-kernel Threefry (examples/03_sde_montecarlo.py:97-119) */
/* drift_dt and vol_sqdt arrive as the float32 values the kernel body forms.   */
/* ------------------------------------------------------------------------- */
ORC_API void orc_gbm(int64_t n, const uint32_t* key, int64_t path_offset, int64_t steps, float s0, float strike,
                     float drift_dt, float vol_sqdt, float* terminal, float* payoff) {
    const float two_pi = (float)(2.0 * 3.141592653589793);
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < n; ++p) {
        uint32_t key0[2];
        threefry(key[0], key[1], 0u, (uint32_t)(path_offset + p), &key0[0], &key0[1]);
        float s = s0;
        for (int64_t i = 0; i < steps; ++i) {
            uint32_t ka[2], kb[2];
            threefry(key0[0], key0[1], 0u, (uint32_t)(2 * i), &ka[0], &ka[1]);
            threefry(key0[0], key0[1], 0u, (uint32_t)(2 * i + 1), &kb[0], &kb[1]);
            float u1 = bits_to_uniform(random_bits_at(ka[0], ka[1], 0u));
            u1 = u1 > 1e-7f ? u1 : 1e-7f;
            float u2 = bits_to_uniform(random_bits_at(kb[0], kb[1], 0u));
            float z = sqrtf(-2.0f * logf(u1)) * cosf(two_pi * u2);
            s = s * expf(drift_dt + vol_sqdt * z);
        }
        if (terminal) terminal[p] = s;
        if (payoff) { float d = s - strike; payoff[p] = d > 0.0f ? d : 0.0f; }
    }
}

/* ------------------------------------------------------------------------- */
/* The hand-written GBM kernel with pcg_hash (examples/03_sde_montecarlo.py:34-70) */
/* ------------------------------------------------------------------------- */
static uint32_t pcg_hash(uint32_t v) {
    uint32_t state = v * 747796405u + 2891336453u;
    uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}
static float pcg_uniform01(uint32_t v) { return ((float)pcg_hash(v) + 0.5f) * 2.3283064e-10f; }

ORC_API void orc_pcg_hash(int64_t n, uint32_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = pcg_hash((uint32_t)i);
}

ORC_API void orc_gbm_pcg(int64_t n, int64_t path_offset, int64_t steps, float s0, float strike, float drift_dt,
                         float vol_sqdt, float* terminal, float* payoff) {
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < n; ++p) {
        const uint32_t tid = (uint32_t)(path_offset + p);
        float s = s0;
        for (uint32_t i = 0; i < (uint32_t)steps; ++i) {
            uint32_t ctr = tid * (uint32_t)steps + i;
            float u1 = pcg_uniform01(2u * ctr);
            float u2 = pcg_uniform01(2u * ctr + 1u);
            float z = sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
            s *= expf(drift_dt + vol_sqdt * z);
        }
        if (terminal) terminal[p] = s;
        if (payoff) { float d = s - strike; payoff[p] = d > 0.0f ? d : 0.0f; }
    }
}

/* ------------------------------------------------------------------------- */
/* Gray-Scott stencil step (examples/04_reaction_diffusion.py:61-74), periodic  */
/* ------------------------------------------------------------------------- */
static void gray_scott_step(int64_t rows, int64_t cols, const float* u_, const float* v_, float* uo, float* vo,
                            float DU, float DV, float F, float FK, float DT) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i) {
        const int64_t ip = (i == rows - 1) ? 0 : i + 1, im = (i == 0) ? rows - 1 : i - 1;
        for (int64_t j = 0; j < cols; ++j) {
            const int64_t jp = (j == cols - 1) ? 0 : j + 1, jm = (j == 0) ? cols - 1 : j - 1;
            const float u = u_[i * cols + j], v = v_[i * cols + j];
            const float lap_u = (((u_[ip * cols + j] + u_[im * cols + j]) + u_[i * cols + jp]) + u_[i * cols + jm]) - 4.0f * u;
            const float lap_v = (((v_[ip * cols + j] + v_[im * cols + j]) + v_[i * cols + jp]) + v_[i * cols + jm]) - 4.0f * v;
            const float uvv = (u * v) * v;
            uo[i * cols + j] = u + DT * ((DU * lap_u - uvv) + F * (1.0f - u));
            vo[i * cols + j] = v + DT * ((DV * lap_v + uvv) - FK * v);
        }
    }
}

ORC_API int orc_gray_scott(int64_t rows, int64_t cols, const float* u, const float* v, float* uo, float* vo,
                           double du, double dv, double f, double k, double dt, int64_t steps) {
    const size_t bytes = (size_t)rows * (size_t)cols * sizeof(float);
    float* a_u = (float*)malloc(bytes); float* a_v = (float*)malloc(bytes);
    float* b_u = (float*)malloc(bytes); float* b_v = (float*)malloc(bytes);
    if (!a_u || !a_v || !b_u || !b_v) { free(a_u); free(a_v); free(b_u); free(b_v); return 1; }
    memcpy(a_u, u, bytes); memcpy(a_v, v, bytes);
    const float DU = (float)du, DV = (float)dv, F = (float)f, FK = (float)(f + k), DT = (float)dt;
    for (int64_t s = 0; s < steps; ++s) {
        gray_scott_step(rows, cols, a_u, a_v, b_u, b_v, DU, DV, F, FK, DT);
        float* t;
        t = a_u; a_u = b_u; b_u = t;
        t = a_v; a_v = b_v; b_v = t;
    }
    memcpy(uo, a_u, bytes); memcpy(vo, a_v, bytes);
    free(a_u); free(a_v); free(b_u); free(b_v);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* df32 arithmetic, restated from the textbook definitions.                    */
/* ------------------------------------------------------------------------- */
#include "df32_ops.h"

/* elementwise df32 primitives, for exactness tests: op 0 add, 1 sub, 2 mul, 3 div, 4 sqrt(a), 5 1/a, 6 1/sqrt(a) */
ORC_API void orc_df_op(int op, int64_t n, const float* ah, const float* al, const float* bh, const float* bl,
                       float* oh, float* ol) {
    for (int64_t i = 0; i < n; ++i) {
        df a = {ah[i], al[i]}, b = {bh[i], bl[i]}, r;
        switch (op) {
            case 0: r = df_add(a, b); break;
            case 1: r = df_sub(a, b); break;
            case 2: r = df_mul(a, b); break;
            case 3: r = df_div(a, b); break;
            case 5: r = df_recip(a); break;
            case 6: r = df_rsqrt(a); break;
            default: r = df_sqrt(a); break;
        }
        oh[i] = r.hi; ol[i] = r.lo;
    }
}
/* error-free transforms on their own: op 0 two_sum, 1 two_prod */
ORC_API void orc_eft(int op, int64_t n, const float* a, const float* b, float* hi, float* lo) {
    for (int64_t i = 0; i < n; ++i) {
        df r = op == 0 ? two_sum(a[i], b[i]) : two_prod(a[i], b[i]);
        hi[i] = r.hi; lo[i] = r.lo;
    }
}

/* df32 RK4 Lotka-Volterra (examples/05_df32_precision.py:27-80) */
ORC_API void orc_lv_rk4_df32(int64_t n, const float* x0, const float* y0, const float* a_, const float* b_,
                             const float* c_, const float* d_, float* xo, float* yo, double dt_, int64_t steps) {
    const float dt = (float)dt_;
    const df half_dt = dfc(0.5f * dt), full_dt = dfc(dt), sixth_dt = dfc(dt / 6.0f), two = dfc(2.0f);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const df a = dfc(a_[i]), b = dfc(b_[i]), c = dfc(c_[i]), d = dfc(d_[i]);
        df x = dfc(x0[i]), y = dfc(y0[i]);
        for (int64_t s = 0; s < steps; ++s) {
            df kx[4], ky[4], sx = x, sy = y;
            for (int st = 0; st < 4; ++st) {
                df xy = df_mul(sx, sy);
                kx[st] = df_sub(df_mul(a, sx), df_mul(b, xy));
                ky[st] = df_sub(df_mul(c, xy), df_mul(d, sy));
                if (st < 3) {
                    df h = st == 2 ? full_dt : half_dt;
                    sx = df_add(x, df_mul(h, kx[st]));
                    sy = df_add(y, df_mul(h, ky[st]));
                }
            }
            df sumx = df_add(df_add(df_add(kx[0], df_mul(two, kx[1])), df_mul(two, kx[2])), kx[3]);
            df sumy = df_add(df_add(df_add(ky[0], df_mul(two, ky[1])), df_mul(two, ky[2])), ky[3]);
            x = df_add(x, df_mul(sixth_dt, sumx));
            y = df_add(y, df_mul(sixth_dt, sumy));
        }
        xo[i] = x.hi + x.lo; yo[i] = y.hi + y.lo;
    }
}

/* df32 RK4 Kepler orbits: r' = v, v' = -GM r / |r|^3; state and result as (hi, lo) */
static inline df split_double(double v) { df r; r.hi = (float)v; r.lo = (float)(v - (double)r.hi); return r; }

ORC_API void orc_kepler_rk4_df32(int64_t n, const float* const* in, float* const* out, double dt_, double gm_,
                                 int64_t steps) {
    const df dt = split_double(dt_), gm = split_double(gm_);
    df half_dt; half_dt.hi = 0.5f * dt.hi; half_dt.lo = 0.5f * dt.lo;
    const df sixth_dt = df_div(dt, dfc(6.0f));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        df s[4];
        for (int c = 0; c < 4; ++c) { s[c].hi = in[2 * c][i]; s[c].lo = in[2 * c + 1][i]; }
        for (int64_t it = 0; it < steps; ++it) {
            df k[4][4], w[4];
            for (int c = 0; c < 4; ++c) w[c] = s[c];
            for (int st = 0; st < 4; ++st) {
                df r2 = df_add(df_mul(w[0], w[0]), df_mul(w[1], w[1]));
                df rs = df_rsqrt(r2);                    /* 1 / |r| */
                df g = df_mul(df_mul(rs, rs), rs);       /* 1 / |r|^3 */
                if (!(gm.hi == 1.0f && gm.lo == 0.0f)) g = df_mul(gm, g);
                k[st][0] = w[2];
                k[st][1] = w[3];
                k[st][2] = df_neg(df_mul(w[0], g));
                k[st][3] = df_neg(df_mul(w[1], g));
                if (st < 3) {
                    df h = st == 2 ? dt : half_dt;
                    for (int c = 0; c < 4; ++c) w[c] = df_add(s[c], df_mul(h, k[st][c]));
                }
            }
            for (int c = 0; c < 4; ++c) {
                df sum = df_add(df_add(df_add(k[0][c], df_twice(k[1][c])), df_twice(k[2][c])), k[3][c]);
                s[c] = df_add(s[c], df_mul(sixth_dt, sum));
            }
        }
        for (int c = 0; c < 4; ++c) { out[2 * c][i] = s[c].hi; out[2 * c + 1][i] = s[c].lo; }
    }
}

/* float64 RK4 Kepler: the truth the df32 result is measured against */
ORC_API void orc_kepler_rk4_f64(int64_t n, const double* in, double* out, double dt, double gm, int64_t steps) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        double s[4] = {in[4 * i], in[4 * i + 1], in[4 * i + 2], in[4 * i + 3]};
        for (int64_t it = 0; it < steps; ++it) {
            double k[4][4], w[4] = {s[0], s[1], s[2], s[3]};
            for (int st = 0; st < 4; ++st) {
                double r2 = w[0] * w[0] + w[1] * w[1];
                double r = sqrt(r2);
                double g = gm / (r2 * r);
                k[st][0] = w[2]; k[st][1] = w[3]; k[st][2] = -(w[0] * g); k[st][3] = -(w[1] * g);
                if (st < 3) {
                    double h = st == 2 ? dt : 0.5 * dt;
                    for (int c = 0; c < 4; ++c) w[c] = s[c] + h * k[st][c];
                }
            }
            for (int c = 0; c < 4; ++c) s[c] = s[c] + dt / 6.0 * (k[0][c] + 2 * k[1][c] + 2 * k[2][c] + k[3][c]);
        }
        for (int c = 0; c < 4; ++c) out[4 * i + c] = s[c];
    }
}

/* float32 RK4 Kepler, plain arithmetic: shows what df32 buys (examples/05's FAST/SAFE rows) */
ORC_API void orc_kepler_rk4_f32(int64_t n, const float* in, float* out, double dt_, double gm_, int64_t steps) {
    const float dt = (float)dt_, gm = (float)gm_, hdt = (float)(0.5 * dt_), sdt = (float)(dt_ / 6.0);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float s[4] = {in[4 * i], in[4 * i + 1], in[4 * i + 2], in[4 * i + 3]};
        for (int64_t it = 0; it < steps; ++it) {
            float k[4][4], w[4] = {s[0], s[1], s[2], s[3]};
            for (int st = 0; st < 4; ++st) {
                float r2 = w[0] * w[0] + w[1] * w[1];
                float r = sqrtf(r2);
                float g = gm / (r2 * r);
                k[st][0] = w[2]; k[st][1] = w[3]; k[st][2] = -(w[0] * g); k[st][3] = -(w[1] * g);
                if (st < 3) {
                    float h = st == 2 ? dt : hdt;
                    for (int c = 0; c < 4; ++c) w[c] = s[c] + h * k[st][c];
                }
            }
            for (int c = 0; c < 4; ++c)
                s[c] = s[c] + sdt * (((k[0][c] + 2.0f * k[1][c]) + 2.0f * k[2][c]) + k[3][c]);
        }
        for (int c = 0; c < 4; ++c) out[4 * i + c] = s[c];
    }
}

/* the deterministic pow, exposed so tests can compare it with double pow */
ORC_API void orc_pd_powf(int64_t n, const float* x, const float* y, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = pd_powf(x[i], y[i]);
}

/* the controller-grade power (1 / err) ** c, exposed for the same purpose */
ORC_API void orc_pd_ctrl_pow(int64_t n, const float* err, const float* c, float* out) {
    for (int64_t i = 0; i < n; ++i) { float unused; pd_ctrl_powers(err[i], c[i], c[i], &out[i], &unused); }
}

/* The C library's float functions on arrays, for the NumPy stand-in that runs the
 * reference's Pallas kernel bodies (tests/golden/pallas_numpy.py): NumPy's own
 * float32 loops for these functions round differently from the C library.
 * op: 0 powf(x, y[i]), 1 expf, 2 logf, 3 cosf, 4 sqrtf. */
ORC_API void orc_libm_f32(int op, int64_t n, const float* x, const float* y, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        switch (op) {
            case 0: out[i] = powf(x[i], y[i]); break;
            case 1: out[i] = expf(x[i]); break;
            case 2: out[i] = logf(x[i]); break;
            case 3: out[i] = cosf(x[i]); break;
            default: out[i] = sqrtf(x[i]); break;
        }
    }
}

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
