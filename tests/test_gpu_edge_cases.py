"""Edge cases the reference singles out: NaN / Inf are well defined under SAFE
and RELAXED (tests/test_07_preflight.py:5-9 in the reference), empty and
degenerate launches, and the inputs that take a kernel's alternative code path."""

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from palladium_b200 import workloads as W
from tests import helpers as H

pytestmark = pytest.mark.gpu
SAFE, RELAXED, FAST = pd.MathMode.SAFE, pd.MathMode.RELAXED, pd.MathMode.FAST


def test_lv_nan_inf_and_zero_parameters_safe():
    n = 64
    args = [a.copy() for a in W.lotka_volterra_ensemble(n)]
    args[0][0] = np.nan
    args[1][1] = np.inf
    args[2][2] = 0.0
    args[3][3] = 0.0       # b = 0
    args[4][4] = 0.0       # c = 0
    args[5][5] = -np.inf
    args[0][6] = 1e30      # overflows within a few steps
    got = H.lv_solver(n, steps=200, math_mode=SAFE)(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=200)
    np.testing.assert_array_equal(got[0], want[0])  # NaNs compare equal position by position
    np.testing.assert_array_equal(got[1], want[1])
    assert np.isnan(got[0][0]) and np.isfinite(got[0][8:]).all()


@pytest.mark.parametrize("mode", [RELAXED, FAST])
def test_lv_degenerate_parameters_take_the_unscaled_path(mode):
    """FAST integrates the rescaled state (c x, b y); b or c that are zero, tiny
    or huge must fall back to the plain form and still agree with the oracle."""
    n = 4096
    args = [a.copy() for a in W.lotka_volterra_ensemble(n)]
    args[3][::7] = 0.0          # b = 0: prey grows exponentially, dx = a x
    args[4][3::11] = 0.0        # c = 0: predators decay, dy = -d y
    args[3][5::13] = 1e-25      # tiny b
    steps = 300
    got = H.lv_solver(n, steps=steps, math_mode=mode)(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=steps)
    # exponentially growing populations (b = 0) amplify per-step rounding: 4e-5 measured
    np.testing.assert_allclose(got[0], want[0], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-4, atol=1e-6)


def test_adaptive_non_finite_lanes_run_the_full_budget_like_the_oracle():
    n = 96
    x0, v0, mu = (a.copy() for a in W.van_der_pol_ensemble(n))
    x0[0] = np.nan
    mu[1] = 1e30        # overflows to inf/NaN on the first attempts
    v0[2] = np.inf
    x0[3], v0[3] = 0.0, 0.0   # the fixed point: error estimate is exactly zero every step
    mu[4] = 0.0
    cfg = dict(t1=2.0, rtol=1e-5, atol=1e-7, dt0=1e-2, max_steps=700)
    got = H.vdp_solver(n, outputs=6, math_mode=SAFE, **cfg)(x0, v0, mu)
    want = oracle.vdp_bs32(x0, v0, mu, pow="pd", **cfg)
    for g, w, name in zip(got, want, ("t", "x", "v", "steps", "rejected", "real")):
        np.testing.assert_array_equal(g, w, err_msg=name)
    assert got[4][0] == cfg["max_steps"]          # a NaN lane rejects every attempt
    assert got[0][3] == np.float32(cfg["t1"])     # the fixed point still reaches t1


def test_adaptive_budget_exhaustion_matches_oracle():
    n = 257
    x0, v0, mu = W.van_der_pol_ensemble(n)
    cfg = dict(t1=20.0, rtol=1e-6, atol=1e-8, dt0=1e-3, max_steps=300)  # far too few steps
    got = H.vdp_solver(n, outputs=6, math_mode=SAFE, **cfg)(x0, v0, mu)
    want = oracle.vdp_bs32(x0, v0, mu, pow="pd", **cfg)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    assert (got[0] < 20.0).all() and (got[3] + got[4] == 300).all()


def test_adaptive_zero_budget_and_zero_trajectories():
    x0, v0, mu = W.van_der_pol_ensemble(5)
    t, x, v, steps, rejected, real = H.vdp_solver(5, outputs=6, math_mode=SAFE, max_steps=0)(x0, v0, mu)
    np.testing.assert_array_equal(x, x0)
    assert (t == 0).all() and (steps == 0).all() and (real == 0).all()
    empty = np.zeros(0, np.float32)
    out = H.vdp_solver(0, outputs=3, math_mode=SAFE)(empty, empty, empty)
    assert out[0].shape == (0, 2) and out[1].shape == (0,)


def test_gbm_zero_steps_and_zero_paths():
    key = W.gbm_key(0)
    terminal, sums = H.gbm_solver(100, with_sums=True, output="terminal", steps=0, s0=123.0, strike=100.0)(key)
    assert (terminal == np.float32(123.0)).all()
    np.testing.assert_allclose(sums, [100 * 23.0, 100 * 23.0 ** 2])
    out, sums = H.gbm_solver(0, with_sums=True, steps=4)(key)
    assert out.shape == (0,) and (sums == 0).all()


def test_gray_scott_nan_spreads_one_cell_per_step_like_the_oracle():
    size = 128
    u, v = W.gray_scott_initial_state(size, patches=2, patch=16)
    u[5, 127] = np.nan       # on the periodic seam
    v[64, 0] = np.inf
    for steps in (1, 4, 6):
        got = H.gs_solver(size, size, math_mode=SAFE, steps=steps)(u, v)
        want = oracle.gray_scott(u, v, steps=steps)
        np.testing.assert_array_equal(got[0], want[0])
        np.testing.assert_array_equal(got[1], want[1])
    assert np.isnan(got[0]).sum() > 50 and np.isfinite(got[0][40, 60])


def test_gray_scott_zero_steps_copies():
    u, v = W.gray_scott_initial_state(64, patches=1, patch=8)
    got = H.gs_solver(64, 64, steps=0)(u, v)
    np.testing.assert_array_equal(got[0], u)
    np.testing.assert_array_equal(got[1], v)


def test_df32_non_finite_inputs_match_the_oracle():
    n = 32
    args = [a.copy() for a in W.lotka_volterra_ensemble(n)]
    args[0][0] = np.nan
    args[1][1] = np.inf
    got = H.lv_solver(n, steps=20, df32=True, math_mode=SAFE)(*args)
    want = oracle.lv_rk4_df32(*args, dt=0.01, steps=20)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])


# The SAFE adaptive kernels divide with pd_div_nonneg, a correctly rounded sequence
# without the compiler's data-dependent slow path; every quotient must equal the
# IEEE division's bit for bit.  A caller-written kernel (pd_math.h is in scope)
# compares the two on the device: per thread REPS operand pairs drawn from Threefry
# bits, the mismatches counted.
DIV_CHECK = r'''
extern "C" __global__ void div_check(const uint32_t* key, const uint32_t* range, uint32_t* bad,
                                     long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    const pd_u32x2 k = pd_fold_in(key[0], key[1], (uint32_t)i);
    // exponent fields: a in [range[0], range[0] + range[1]), b in [range[2], range[2] + range[3])
    const uint32_t a_lo = range[0], a_n = range[1], b_lo = range[2], b_n = range[3], reps = range[4];
    uint32_t count = 0;
    for (uint32_t rep = 0; rep < reps; ++rep) {
        const uint32_t ra = pd_random_bits(k.a, k.b, 3u * rep), rb = pd_random_bits(k.a, k.b, 3u * rep + 1u);
        const uint32_t rc = pd_random_bits(k.a, k.b, 3u * rep + 2u);
        uint32_t ma = ra & 0x007FFFFFu, mb = rb & 0x007FFFFFu;
        // one pair in four gets a significand that is hard for division: all ones, a single bit, or zero
        if ((rc & 3u) == 0u) ma = (rc & 4u) ? 0x007FFFFFu : ((rc & 8u) ? 0u : 1u << ((rc >> 8) % 23u));
        if ((rc & 48u) == 0u) mb = (rc & 64u) ? 0x007FFFFFu : ((rc & 128u) ? 0u : 1u << ((rc >> 16) % 23u));
        const float a = pd_u2f(((a_lo + (ra >> 23) % a_n) << 23) | ma);
        const float b = pd_u2f(((b_lo + (rb >> 23) % b_n) << 23) | mb);
        count += pd_f2u(pd_div_nonneg(a, b)) != pd_f2u(__fdiv_rn(a, b)) ? 1u : 0u;
        // the two-quotient form (packed instructions), this pair next to the swapped-significand one
        const float a2 = pd_u2f(((a_lo + (rb >> 23) % a_n) << 23) | mb), b2 = pd_u2f(((b_lo + (ra >> 23) % b_n) << 23) | ma);
        float q1, q2;
        pd_div_nonneg_pair(a, b, a2, b2, &q1, &q2);
        count += pd_f2u(q1) != pd_f2u(__fdiv_rn(a, b)) ? 1u : 0u;
        count += pd_f2u(q2) != pd_f2u(__fdiv_rn(a2, b2)) ? 1u : 0u;
    }
    // the special values, once per thread: zero numerators, and operands outside the stated range
    const float special[8] = {0.0f, 1e-42f, 3e38f, 1.0f, pd_u2f(0x7F800000u), pd_u2f(0x7FC00000u), -1.0f, 1e-30f};
    for (int p = 0; p < 8; ++p)
        for (int q = 0; q < 8; ++q) {
            const uint32_t want = pd_f2u(__fdiv_rn(special[p], special[q])), got = pd_f2u(pd_div_nonneg(special[p], special[q]));
            const bool both_nan = (want & 0x7FFFFFFFu) > 0x7F800000u && (got & 0x7FFFFFFFu) > 0x7F800000u;
            count += (want != got && !both_nan) ? 1u : 0u;
            float q1, q2;   // a special value beside an ordinary quotient sends both down the scalar path
            pd_div_nonneg_pair(special[p], special[q], 3.0f, 7.0f, &q1, &q2);
            const bool nan1 = (want & 0x7FFFFFFFu) > 0x7F800000u && (pd_f2u(q1) & 0x7FFFFFFFu) > 0x7F800000u;
            count += (want != pd_f2u(q1) && !nan1) ? 1u : 0u;
            count += pd_f2u(q2) != pd_f2u(__fdiv_rn(3.0f, 7.0f)) ? 1u : 0u;
        }
    bad[i] = count;
}
'''


@pytest.mark.parametrize("name,a_lo,a_n,b_lo,b_n", [
    ("the whole stated range: a in [2^-104, 2^60), b in [2^-60, 2^20)", 23, 164, 67, 80),
    ("error-norm operands: a in [2^-50, 2^-10), b in [2^-30, 2^-5)", 77, 40, 97, 25),
    ("beyond the range on both sides (the IEEE division itself)", 1, 253, 1, 253),
])
def test_safe_division_equals_ieee_division_bit_for_bit(name, a_lo, a_n, b_lo, b_n):
    from palladium_b200 import families, pl

    threads, reps = 1 << 20, 2048        # 2.1e9 operand pairs per case
    call = pd.cuda_call(families.source_kernel(DIV_CHECK, "div_check"), grid=(threads,),
                        out_shape=pl.ShapeDtypeStruct((threads,), np.uint32), math_mode=SAFE)
    bad = call(W.gbm_key(11), np.array([a_lo, a_n, b_lo, b_n, reps], np.uint32))
    assert int(bad.sum()) == 0, f"{int(bad.sum())} of {threads * reps} quotients differ: {name}"


CTRL_POW = r'''
extern "C" __global__ void ctrl_pow(const float* err, const float* c, float* r1, float* r2,
                                    long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    pd_ctrl_powers(err[i], c[0], c[1], &r1[i], &r2[i]);
}
'''


def test_controller_powers_on_the_device_equal_the_host_routine_bit_for_bit():
    """The device evaluates the controller's two powers on packed instructions, the CPU oracle one
    after the other: every bit must agree, the integer step counts depend on it.  Two million error
    norms over the range the controller sees and beyond it, the special values included."""
    from palladium_b200 import families, pl

    rng = np.random.default_rng(8)
    err = np.concatenate([np.exp(rng.uniform(np.log(1e-9), np.log(1e9), 1 << 21)).astype(np.float32),
                          np.exp(rng.uniform(np.log(1e-38), np.log(1e38), 1 << 18)).astype(np.float32),
                          np.array([0.0, np.inf, np.nan, 1e-42, 1.0, 1e-9, -1.0], np.float32)])
    n = err.size
    sh = pl.ShapeDtypeStruct((n,), np.float32)
    call = pd.cuda_call(families.source_kernel(CTRL_POW, "ctrl_pow"), grid=(n,), out_shape=(sh, sh), math_mode=SAFE)
    for c1, c2 in ((0.7 / 3, -0.4 / 3), (0.7 / 5, -0.4 / 5), (0.5, -0.25), (20.0, -20.0)):
        coeff = np.array([c1, c2], np.float32)
        r1, r2 = call(err, coeff)
        np.testing.assert_array_equal(r1.view(np.uint32)[:-5], oracle.pd_ctrl_pow(err, coeff[0]).view(np.uint32)[:-5])
        np.testing.assert_array_equal(r2.view(np.uint32)[:-5], oracle.pd_ctrl_pow(err, coeff[1]).view(np.uint32)[:-5])
        np.testing.assert_array_equal(r1, oracle.pd_ctrl_pow(err, coeff[0]))      # NaN where the host has NaN
        np.testing.assert_array_equal(r2, oracle.pd_ctrl_pow(err, coeff[1]))
