"""Run-time right-hand sides on the GPU (NVRTC-compiled kernels) against the
oracle built from the same source text, and against the hand-written families
for the two systems both can express.  Follows the reference's rule for new
lowering rules (docs/extending.md:51-69): diff against the oracle, then break
the kernel on purpose and see the test fail."""

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from oracle import custom_ode as oracle_custom
from palladium_b200 import workloads as W

from tests import helpers as H

pytestmark = pytest.mark.gpu

SAFE, RELAXED, FAST = pd.MathMode.SAFE, pd.MathMode.RELAXED, pd.MathMode.FAST
LV = "dy[0] = p[0]*y[0] - (p[1]*y[0])*y[1];\ndy[1] = (p[2]*y[0])*y[1] - p[3]*y[1];"
VDP = "dy[0] = y[1];\ndy[1] = (p[0]*(1.0f - y[0]*y[0]))*y[1] - y[0];"
LORENZ = ("dy[0] = p[0]*(y[1] - y[0]);\n"
          "dy[1] = y[0]*(p[1] - y[2]) - y[1];\n"
          "dy[2] = y[0]*y[1] - p[2]*y[2];")
FORCED = "dy[0] = y[1];\ndy[1] = (p[1]*sinf(p[2]*t) - p[0]*y[1]) - y[0];"
VDP_CFG = dict(t1=2.0, rtol=1e-5, atol=1e-7, dt0=0.01, max_steps=3000)


def lorenz_ensemble(n, seed=23):
    rng = np.random.default_rng(seed)
    state = [rng.uniform(-5, 5, n).astype(np.float32) for _ in range(3)]
    params = [rng.uniform(9, 11, n).astype(np.float32), rng.uniform(20, 30, n).astype(np.float32),
              rng.uniform(2.0, 3.0, n).astype(np.float32)]
    return state + params


@pytest.mark.parametrize("n", [1, 1000, 4099])
def test_lotka_volterra_source_reproduces_the_hand_written_family_bit_for_bit(n):
    ins = W.lotka_volterra_ensemble(n)
    got = H.custom_solver(n, LV, 2, 4, dt=0.01, steps=300)(*ins)
    family = H.lv_solver(n, dt=0.01, steps=300, math_mode=SAFE)(*ins)
    want = oracle.lv_rk4(*ins, dt=0.01, steps=300)
    for g, f, w in zip(got, family, want):
        np.testing.assert_array_equal(g, f)
        np.testing.assert_array_equal(g, w)


def test_van_der_pol_source_reproduces_the_adaptive_family_bit_for_bit():
    n = 2000
    x0, v0, mu = W.van_der_pol_ensemble(n)
    got = H.custom_solver(n, VDP, 2, 1, method="bs32", **VDP_CFG)(x0, v0, mu)
    family = H.vdp_solver(n, outputs=6, math_mode=SAFE, **VDP_CFG)(x0, v0, mu)
    want = oracle.vdp_bs32(x0, v0, mu, pow="pd", **VDP_CFG)
    for g, f, w, name in zip(got, family, want, ("t", "x", "v", "steps", "rejected", "real")):
        np.testing.assert_array_equal(g, f, err_msg=name)
        np.testing.assert_array_equal(g, w, err_msg=name)
    assert np.std(got[5]) > 0


def test_a_system_no_family_covers_lorenz_rk4_and_adaptive():
    n = 3000
    ins = lorenz_ensemble(n)
    got = H.custom_solver(n, LORENZ, 3, 3, dt=0.005, steps=400)(*ins)
    want = oracle_custom.rk4(LORENZ, 3, 3, ins, dt=0.005, steps=400)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    cfg = dict(t1=1.0, rtol=1e-5, atol=1e-7, dt0=0.001, max_steps=4000)
    got = H.custom_solver(n, LORENZ, 3, 3, method="bs32", **cfg)(*ins)
    want = oracle_custom.bs32(LORENZ, 3, 3, ins, pow="pd", **cfg)
    assert len(got) == 7
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    assert np.all(got[0] == 1.0)


@pytest.mark.parametrize("mode", [RELAXED, FAST])
def test_relaxed_and_fast_stay_within_float32_tolerance(mode):
    n = 3000
    ins = lorenz_ensemble(n)
    got = H.custom_solver(n, LORENZ, 3, 3, math_mode=mode, dt=0.005, steps=100)(*ins)
    want = oracle_custom.rk4(LORENZ, 3, 3, ins, dt=0.005, steps=100)
    for g, w in zip(got, want):
        np.testing.assert_allclose(g, w, rtol=2e-4, atol=2e-4)   # 100 steps of a chaotic system amplify rounding


def test_time_dependent_right_hand_side_with_a_library_function():
    n = 2048
    rng = np.random.default_rng(5)
    ins = [rng.uniform(-1, 1, n).astype(np.float32), rng.uniform(-1, 1, n).astype(np.float32),
           rng.uniform(0.1, 0.5, n).astype(np.float32), rng.uniform(0.5, 1.5, n).astype(np.float32),
           rng.uniform(0.5, 2.0, n).astype(np.float32)]
    want = oracle_custom.rk4(FORCED, 2, 3, ins, dt=0.01, steps=500)
    for mode in (SAFE, FAST):
        got = H.custom_solver(n, FORCED, 2, 3, math_mode=mode, dt=0.01, steps=500)(*ins)
        for g, w in zip(got, want):
            np.testing.assert_allclose(g, w, rtol=1e-4, atol=1e-5)   # sinf differs from libm by an ulp or two


def test_broken_on_purpose_the_comparison_fails():
    n = 512
    ins = lorenz_ensemble(n)
    sabotaged = LORENZ.replace("- y[1];", ";")          # drop a term
    got = H.custom_solver(n, sabotaged, 3, 3, dt=0.005, steps=50)(*ins)
    want = oracle_custom.rk4(LORENZ, 3, 3, ins, dt=0.005, steps=50)
    assert not np.allclose(got[1], want[1], rtol=1e-3, atol=1e-3)


def test_large_host_call_takes_the_chunked_pipeline_and_equals_the_device_call():
    import torch

    n = (1 << 18) + 777
    ins = W.lotka_volterra_ensemble(n)
    jit = H.custom_solver(n, LV, 2, 4, call=pd.cuda_call_jit, math_mode=FAST, dt=0.01, steps=50)
    host = jit(*ins)
    dev = jit(*[torch.from_numpy(a).cuda() for a in ins])
    for h, d in zip(host, dev):
        np.testing.assert_array_equal(h, d.cpu().numpy())
    want = oracle.lv_rk4(*ins, dt=0.01, steps=50)
    np.testing.assert_allclose(host[0], want[0], rtol=1e-5, atol=1e-6)


def test_compile_error_at_first_launch_when_the_check_was_skipped():
    from palladium_b200 import families, pl

    n = 32
    fam = families.custom_ode("dy[0] = undefined_name;", 1, check=False)
    call = pd.cuda_call(fam, grid=(n,), out_shape=pl.ShapeDtypeStruct((n,), np.float32))
    with pytest.raises(pd.EmitError, match="undefined_name"):
        call(np.zeros(n, np.float32))


def test_explain_reports_the_compiled_kernel():
    n = 4096
    call = H.custom_solver(n, LORENZ, 3, 3, math_mode=FAST, dt=0.005, steps=10)
    info = call.explain(*lorenz_ensemble(n))
    text = str(info)
    assert "pd_ode_rk4" in text
    assert info.regs > 0 and info.blocks_per_sm > 0 and info.msl_lines == 3


def test_concurrent_first_calls_compile_once_and_agree():
    """Sixteen threads hit a source text nobody has compiled yet (the reference's
    robustness test does the same with a fresh kernel, tests/test_17_robustness.py:22-78):
    the native cache is mutex-guarded, every thread gets the same results."""
    import threading

    n = 2048
    ins = lorenz_ensemble(n, seed=77)
    rhs = LORENZ + "\n// concurrent-first-call variant"       # a text no other test has compiled
    call = H.custom_solver(n, rhs, 3, 3, dt=0.004, steps=64)
    want = oracle_custom.rk4(LORENZ, 3, 3, ins, dt=0.004, steps=64)
    results, errors = [None] * 16, []

    def work(i):
        try:
            results[i] = call(*ins)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(16)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    assert len(call.cache) == 1
    for got in results:
        for g, w in zip(got, want):
            np.testing.assert_array_equal(g, w)


# ------------------------------------------------------------------ the seven-stage 5(4) pairs
@pytest.mark.parametrize("method", ["dopri5", "tsit5"])
def test_adaptive_5_4_pairs_equal_the_oracle_bit_for_bit(method):
    n = 3000
    x0, v0, mu = W.van_der_pol_ensemble(n)
    cfg = dict(t1=2.0, rtol=1e-6, atol=1e-8, dt0=0.01, max_steps=2000)
    got = H.custom_solver(n, VDP, 2, 1, method=method, **cfg)(x0, v0, mu)
    want = oracle_custom.erk(VDP, 2, 1, (x0, v0, mu), method=method, pow="pd", **cfg)
    assert len(got) == 6
    for g, w, name in zip(got, want, ("t", "x", "v", "steps", "rejected", "real")):
        np.testing.assert_array_equal(g, w, err_msg=name)
    assert np.all(got[0] == 2.0) and np.std(got[5]) > 0
    ins = lorenz_ensemble(2000)
    cfg = dict(t1=1.0, rtol=1e-5, atol=1e-7, dt0=0.001, max_steps=2000)
    got = H.custom_solver(2000, LORENZ, 3, 3, method=method, **cfg)(*ins)
    want = oracle_custom.erk(LORENZ, 3, 3, ins, method=method, pow="pd", **cfg)
    assert len(got) == 7
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)


@pytest.mark.parametrize("mode", [RELAXED, FAST])
@pytest.mark.parametrize("method", ["dopri5", "tsit5"])
def test_adaptive_5_4_pairs_relaxed_and_fast(method, mode):
    """The bar the reference sets for its adaptive kernel (tests/test_08_adaptive.py:181-189):
    state within rtol 1e-3, counters within 20."""
    n = 3000
    x0, v0, mu = W.van_der_pol_ensemble(n)
    cfg = dict(t1=2.0, rtol=1e-6, atol=1e-8, dt0=0.01, max_steps=2000)
    got = H.custom_solver(n, VDP, 2, 1, method=method, math_mode=mode, **cfg)(x0, v0, mu)
    want = oracle_custom.erk(VDP, 2, 1, (x0, v0, mu), method=method, pow="pd", **cfg)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_allclose(got[1], want[1], rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(got[2], want[2], rtol=1e-3, atol=1e-5)
    assert np.abs(got[4] - want[4]).max() <= 20 and np.abs(got[5] - want[5]).max() <= 20


def test_a_5_4_pair_takes_fewer_attempts_than_bogacki_shampine():
    n = 3000
    x0, v0, mu = W.van_der_pol_ensemble(n)
    cfg = dict(t1=2.0, rtol=1e-6, atol=1e-8, dt0=0.01, max_steps=3000)
    low = H.custom_solver(n, VDP, 2, 1, method="bs32", **cfg)(x0, v0, mu)
    high = H.custom_solver(n, VDP, 2, 1, method="tsit5", **cfg)(x0, v0, mu)
    assert high[5].mean() < 0.3 * low[5].mean()
    np.testing.assert_allclose(high[1], low[1], rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("method", ["dopri5", "tsit5"])
def test_adaptive_5_4_pairs_edge_cases_follow_the_oracle(method):
    """Non-finite and degenerate lanes (a NaN state rejects every attempt, an overflowing parameter,
    the fixed point whose error estimate is exactly zero), a budget far too small, and a zero budget."""
    n = 96
    x0, v0, mu = (a.copy() for a in W.van_der_pol_ensemble(n))
    x0[0] = np.nan
    mu[1] = 1e30
    v0[2] = np.inf
    x0[3], v0[3] = 0.0, 0.0
    mu[4] = 0.0
    cfg = dict(t1=2.0, rtol=1e-5, atol=1e-7, dt0=1e-2, max_steps=400)
    got = H.custom_solver(n, VDP, 2, 1, method=method, **cfg)(x0, v0, mu)
    want = oracle_custom.erk(VDP, 2, 1, (x0, v0, mu), method=method, pow="pd", **cfg)
    for g, w, name in zip(got, want, ("t", "x", "v", "steps", "rejected", "real")):
        np.testing.assert_array_equal(g, w, err_msg=name)
    assert got[4][0] == cfg["max_steps"] and got[0][3] == np.float32(cfg["t1"])

    x0, v0, mu = W.van_der_pol_ensemble(257)
    cfg = dict(t1=20.0, rtol=1e-6, atol=1e-8, dt0=1e-3, max_steps=40)
    got = H.custom_solver(257, VDP, 2, 1, method=method, **cfg)(x0, v0, mu)
    want = oracle_custom.erk(VDP, 2, 1, (x0, v0, mu), method=method, pow="pd", **cfg)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    assert (got[0] < 20.0).any() and (got[3] + got[4] == 40).all()

    t, x, v, steps, rejected, real = H.custom_solver(257, VDP, 2, 1, method=method, max_steps=0)(x0, v0, mu)
    np.testing.assert_array_equal(x, x0)
    assert (t == 0).all() and (steps == 0).all() and (real == 0).all()


def test_adaptive_5_4_pair_scalar_system_without_parameters():
    n = 1000
    y0 = np.linspace(0.1, 2.0, n).astype(np.float32)
    cfg = dict(t1=1.0, rtol=1e-6, atol=1e-9, dt0=1e-2, max_steps=300)
    got = H.custom_solver(n, "dy[0] = -y[0] * y[0];", 1, 0, method="tsit5", **cfg)(y0)
    want = oracle_custom.erk("dy[0] = -y[0] * y[0];", 1, 0, (y0,), method="tsit5", pow="pd", **cfg)
    assert len(got) == 5
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    np.testing.assert_allclose(got[1], y0 / (1.0 + y0), rtol=5e-6)    # y' = -y^2: y(1) = y0 / (1 + y0)
