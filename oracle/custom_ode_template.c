/* CPU oracle for run-time right-hand sides.  TEST INFRASTRUCTURE ONLY.
 *
 * oracle/custom_ode.py pastes a right-hand side (the same text the CUDA
 * library compiles with NVRTC) at the marker below and builds this file with
 * gcc -O2 -ffp-contract=off, so every float operation rounds once, in source
 * order.  The two loops restate, for a state of ORC_DIM components:
 *   - the fixed-step RK4 loop of the reference's ensemble kernel
 *     (examples/01_ode_ensembles.py:72-91; operation order of
 *     tests/golden/rk4_lotka_volterra.metal:90-94,186,234-258);
 *   - the adaptive Bogacki-Shampine 3(2) loop with PI controller of
 *     examples/02_adaptive_lockstep.py:69-171, run for the full max_steps
 *     iterations as the reference runs it (no early exit here).
 *   - the same adaptive loop around the seven-stage 5(4) pairs of Dormand-Prince
 *     and Tsitouras (coefficients in pd_math.h).  The reference has no kernel
 *     of these, only a CPU comparison that runs diffrax's Tsit5
 *     (benchmarks/bench_ensembles.py:88-118): parity unpinned; what pins the
 *     coefficients is the order conditions and a float64 solution
 *     (tests/test_oracle.py).
 * On the reference's own two systems the first two loops equal the pinned family
 * oracles bit for bit; for other systems parity is unpinned (the reference has
 * nothing to compare with).
 */
#include <stdint.h>
#include <math.h>
#include "pd_math.h"

#ifndef ORC_NPARAM_ALLOC
#define ORC_NPARAM_ALLOC 1
#endif

static inline void user_rhs(float t, const float* y, const float* p, float* dy) {
    (void)t; (void)p;
/*ORC_RHS*/
}

__attribute__((visibility("default")))
void orc_custom_rk4(int64_t n, const float* const* in, float* const* out, int64_t steps, double dt) {
    const float hh = (float)(0.5 * dt), hf = (float)dt, h6 = (float)(dt / 6.0);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float y[ORC_DIM], p[ORC_NPARAM_ALLOC], w[ORC_DIM], k1[ORC_DIM], k2[ORC_DIM], k3[ORC_DIM], k4[ORC_DIM];
        for (int c = 0; c < ORC_DIM; ++c) y[c] = in[c][i];
        for (int c = 0; c < ORC_NPARAM; ++c) p[c] = in[ORC_DIM + c][i];
        for (int64_t s = 0; s < steps; ++s) {
            const float t = (float)s * hf;
            user_rhs(t, y, p, k1);
            for (int c = 0; c < ORC_DIM; ++c) w[c] = y[c] + hh * k1[c];
            user_rhs(t + hh, w, p, k2);
            for (int c = 0; c < ORC_DIM; ++c) w[c] = y[c] + hh * k2[c];
            user_rhs(t + hh, w, p, k3);
            for (int c = 0; c < ORC_DIM; ++c) w[c] = y[c] + hf * k3[c];
            user_rhs(t + hf, w, p, k4);
            for (int c = 0; c < ORC_DIM; ++c)
                y[c] = y[c] + h6 * (((k1[c] + 2.0f * k2[c]) + 2.0f * k3[c]) + k4[c]);
        }
        for (int c = 0; c < ORC_DIM; ++c) out[c][i] = y[c];
    }
}

static inline float max_nan(float a, float b) { return (a != a) ? a : (b != b) ? b : (a > b ? a : b); }
static inline float min_nan(float a, float b) { return (a != a) ? a : (b != b) ? b : (a < b ? a : b); }

/* out: t, ORC_DIM states, steps, rejected, real.  pow_flavour 0: libm powf on 1/err; 1: pd_ctrl_powers on err. */
__attribute__((visibility("default")))
void orc_custom_bs32(int64_t n, const float* const* in, float* const* out, double t1_, double rtol_, double atol_,
                     double dt0_, double pcoeff, double icoeff, double safety_, double fmin_, double fmax_,
                     int64_t error_order, int64_t max_steps, int pow_flavour) {
    const float T1 = (float)t1_, RTOL = (float)rtol_, ATOL = (float)atol_, DT0 = (float)dt0_;
    const float SAFETY = (float)safety_, FMIN = (float)fmin_, FMAX = (float)fmax_;
    const float coeff1 = (float)((icoeff + pcoeff) / (double)error_order);
    const float coeff2 = (float)(-pcoeff / (double)error_order);
    const float c29 = (float)(2.0 / 9.0), c13 = (float)(1.0 / 3.0), c49 = (float)(4.0 / 9.0);
    const float c724 = (float)(7.0 / 24.0), c14 = (float)(1.0 / 4.0), c18 = (float)(1.0 / 8.0);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < n; ++i) {
        float y[ORC_DIM], p[ORC_NPARAM_ALLOC], k1[ORC_DIM], k2[ORC_DIM], k3[ORC_DIM], k4[ORC_DIM], w[ORC_DIM],
            y3[ORC_DIM];
        for (int c = 0; c < ORC_DIM; ++c) y[c] = in[c][i];
        for (int c = 0; c < ORC_NPARAM; ++c) p[c] = in[ORC_DIM + c][i];
        float t = 0.0f, dt = DT0, prev_inv_err = 1.0f, prev_err = 1.0f, steps = 0.0f, rejected = 0.0f, real = 0.0f;
        user_rhs(t, y, p, k1);
        for (int64_t it = 0; it < max_steps; ++it) {
            const int was_real = t < T1;
            dt = min_nan(dt, T1 - t);
            for (int c = 0; c < ORC_DIM; ++c) w[c] = y[c] + (0.5f * dt) * k1[c];
            user_rhs(t + 0.5f * dt, w, p, k2);
            for (int c = 0; c < ORC_DIM; ++c) w[c] = y[c] + (0.75f * dt) * k2[c];
            user_rhs(t + 0.75f * dt, w, p, k3);
            for (int c = 0; c < ORC_DIM; ++c) y3[c] = y[c] + dt * ((c29 * k1[c] + c13 * k2[c]) + c49 * k3[c]);
            user_rhs(t + dt, y3, p, k4);
            float err_norm = 0.0f;
            for (int c = 0; c < ORC_DIM; ++c) {
                const float y2 = y[c] + dt * (((c724 * k1[c] + c14 * k2[c]) + c13 * k3[c]) + c18 * k4[c]);
                const float ratio = fabsf(y3[c] - y2) / (ATOL + RTOL * fabsf(y3[c]));
                err_norm = c == 0 ? ratio : max_nan(err_norm, ratio);
            }
            const int accept = err_norm <= 1.0f;
            if (accept) {
                t = t + dt;
                for (int c = 0; c < ORC_DIM; ++c) { y[c] = y3[c]; k1[c] = k4[c]; }
            }
            err_norm = max_nan(err_norm, 1e-9f);
            const float inv_err = 1.0f / err_norm;
            float pa, pb;
            if (pow_flavour == 1) {
                float unused;
                pd_ctrl_powers(err_norm, coeff1, coeff1, &pa, &unused);
                pd_ctrl_powers(prev_err, coeff2, coeff2, &pb, &unused);
            } else { pa = powf(inv_err, coeff1); pb = powf(prev_inv_err, coeff2); }
            const float factor = (SAFETY * pa) * pb;
            if (accept) { prev_inv_err = inv_err; prev_err = err_norm; }
            dt = dt * min_nan(max_nan(factor, FMIN), FMAX);
            steps = steps + (accept ? 1.0f : 0.0f);
            rejected = rejected + (accept ? 0.0f : 1.0f);
            real = real + ((was_real && accept) ? 1.0f : 0.0f);
        }
        out[0][i] = t;
        for (int c = 0; c < ORC_DIM; ++c) out[1 + c][i] = y[c];
        out[ORC_DIM + 1][i] = steps;
        out[ORC_DIM + 2][i] = rejected;
        out[ORC_DIM + 3][i] = real;
    }
}

/* method 2: Dormand-Prince 5(4); 3: Tsitouras 5(4).  Same outputs and controller as orc_custom_bs32 with
 * pow_flavour as there.  A stage sums its non-zero coefficients left to right. */
__attribute__((visibility("default")))
void orc_custom_erk(int64_t n, const float* const* in, float* const* out, int method, double t1_, double rtol_,
                    double atol_, double dt0_, double pcoeff, double icoeff, double safety_, double fmin_,
                    double fmax_, int64_t error_order, int64_t max_steps, int pow_flavour) {
    static const float A_dp[6][6] = PD_DOPRI5_A, A_ts[6][6] = PD_TSIT5_A;
    static const float C_dp[7] = PD_DOPRI5_C, C_ts[7] = PD_TSIT5_C;
    static const float E_dp[7] = PD_DOPRI5_E, E_ts[7] = PD_TSIT5_E;
    const float (*A)[6] = method == 2 ? A_dp : A_ts;
    const float* C = method == 2 ? C_dp : C_ts;
    const float* E = method == 2 ? E_dp : E_ts;
    const float T1 = (float)t1_, RTOL = (float)rtol_, ATOL = (float)atol_, DT0 = (float)dt0_;
    const float SAFETY = (float)safety_, FMIN = (float)fmin_, FMAX = (float)fmax_;
    const float coeff1 = (float)((icoeff + pcoeff) / (double)error_order);
    const float coeff2 = (float)(-pcoeff / (double)error_order);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < n; ++i) {
        float y[ORC_DIM], p[ORC_NPARAM_ALLOC], k[7][ORC_DIM], w[ORC_DIM];
        for (int c = 0; c < ORC_DIM; ++c) y[c] = in[c][i];
        for (int c = 0; c < ORC_NPARAM; ++c) p[c] = in[ORC_DIM + c][i];
        float t = 0.0f, dt = DT0, prev_inv_err = 1.0f, prev_err = 1.0f, steps = 0.0f, rejected = 0.0f, real = 0.0f;
        user_rhs(t, y, p, k[0]);
        for (int64_t it = 0; it < max_steps; ++it) {
            const int was_real = t < T1;
            dt = min_nan(dt, T1 - t);
            for (int s = 1; s < 7; ++s) {
                for (int c = 0; c < ORC_DIM; ++c) {
                    float acc = A[s - 1][0] * k[0][c];
                    for (int j = 1; j < s; ++j)
                        if (A[s - 1][j] != 0.0f) acc = acc + A[s - 1][j] * k[j][c];
                    w[c] = y[c] + dt * acc;
                }
                user_rhs(t + C[s] * dt, w, p, k[s]);
            }
            float err_norm = 0.0f;
            for (int c = 0; c < ORC_DIM; ++c) {
                float e = E[0] * k[0][c];
                for (int j = 1; j < 7; ++j)
                    if (E[j] != 0.0f) e = e + E[j] * k[j][c];
                const float ratio = fabsf(dt * e) / (ATOL + RTOL * fabsf(w[c]));
                err_norm = c == 0 ? ratio : max_nan(err_norm, ratio);
            }
            const int accept = err_norm <= 1.0f;
            if (accept) {
                t = t + dt;
                for (int c = 0; c < ORC_DIM; ++c) { y[c] = w[c]; k[0][c] = k[6][c]; }
            }
            err_norm = max_nan(err_norm, 1e-9f);
            const float inv_err = 1.0f / err_norm;
            float pa, pb;
            if (pow_flavour == 1) {
                float unused;
                pd_ctrl_powers(err_norm, coeff1, coeff1, &pa, &unused);
                pd_ctrl_powers(prev_err, coeff2, coeff2, &pb, &unused);
            } else { pa = powf(inv_err, coeff1); pb = powf(prev_inv_err, coeff2); }
            const float factor = (SAFETY * pa) * pb;
            if (accept) { prev_inv_err = inv_err; prev_err = err_norm; }
            dt = dt * min_nan(max_nan(factor, FMIN), FMAX);
            steps = steps + (accept ? 1.0f : 0.0f);
            rejected = rejected + (accept ? 0.0f : 1.0f);
            real = real + ((was_real && accept) ? 1.0f : 0.0f);
        }
        out[0][i] = t;
        for (int c = 0; c < ORC_DIM; ++c) out[1 + c][i] = y[c];
        out[ORC_DIM + 1][i] = steps;
        out[ORC_DIM + 2][i] = rejected;
        out[ORC_DIM + 3][i] = real;
    }
}

/* The coefficients as compiled, for the order-condition test. */
__attribute__((visibility("default")))
void orc_tableau(int method, float* a36, float* c7, float* e7) {
    static const float A_dp[6][6] = PD_DOPRI5_A, A_ts[6][6] = PD_TSIT5_A;
    static const float C_dp[7] = PD_DOPRI5_C, C_ts[7] = PD_TSIT5_C;
    static const float E_dp[7] = PD_DOPRI5_E, E_ts[7] = PD_TSIT5_E;
    for (int s = 0; s < 6; ++s)
        for (int j = 0; j < 6; ++j) a36[s * 6 + j] = method == 2 ? A_dp[s][j] : A_ts[s][j];
    for (int j = 0; j < 7; ++j) { c7[j] = method == 2 ? C_dp[j] : C_ts[j]; e7[j] = method == 2 ? E_dp[j] : E_ts[j]; }
}
