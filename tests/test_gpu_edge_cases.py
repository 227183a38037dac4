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
