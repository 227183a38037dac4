"""The benchmark configurations at their full sizes.  The oracle cannot run
these whole, so each is checked through properties that do not depend on size:
a seeded subset against the oracle, closed forms, conservation laws, and
agreement between independent kernel variants."""

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from palladium_b200 import _native
from palladium_b200 import workloads as W
from tests import helpers as H

pytestmark = pytest.mark.gpu
SAFE = pd.MathMode.SAFE


def test_adaptive_one_million_trajectories_subset_matches_oracle():
    cfg = {k: v for k, v in W.VDP_CONFIG.items() if k not in ("n", "seed")}
    n = W.VDP_CONFIG["n"]
    x0, v0, mu = W.van_der_pol_ensemble(n)
    state, accepted, rejected = H.vdp_solver(n, outputs=3, call=pd.cuda_call_jit, math_mode=SAFE, **cfg)(x0, v0, mu)
    assert accepted.min() > 0 and (accepted + rejected).max() < cfg["max_steps"]  # every trajectory reached t1
    pick = np.r_[0:200, 500_000:500_200, n - 200:n]
    want = oracle.vdp_bs32(x0[pick], v0[pick], mu[pick], pow="pd", **cfg)
    np.testing.assert_array_equal(state[pick, 0], want[1])
    np.testing.assert_array_equal(state[pick, 1], want[2])
    np.testing.assert_array_equal(accepted[pick], want[5].astype(np.int32))
    np.testing.assert_array_equal(rejected[pick], want[4].astype(np.int32))
    assert np.all(want[0] == np.float32(cfg["t1"]))


def test_gbm_two_to_the_26_paths_against_black_scholes():
    import torch

    cfg = {k: v for k, v in W.GBM_CONFIG.items() if k not in ("n", "seed")}
    n = W.GBM_CONFIG["n"]
    call = H.gbm_solver(n, with_sums=True, call=pd.cuda_call_jit, output="terminal", **cfg)
    terminal, sums = call(torch.from_numpy(W.gbm_key(0)).cuda())
    s1, s2 = (float(x) for x in sums.cpu())
    disc = np.exp(-cfg["r"] * cfg["t"])
    price = disc * s1 / n
    stderr = disc * np.sqrt((s2 / n - (s1 / n) ** 2) / n)
    exact = oracle.black_scholes_call(cfg["s0"], cfg["strike"], cfg["t"], cfg["r"], cfg["sigma"])
    assert abs(price - exact) < 5 * stderr  # examples/03_sde_montecarlo.py:146
    assert stderr < 2.5e-3
    # the sums are the sums of the per-path payoffs, and the head of the run equals the oracle's paths
    payoff = torch.clamp(terminal - cfg["strike"], min=0.0).double()
    np.testing.assert_allclose(float(payoff.sum()), s1, rtol=1e-9)
    head, _ = oracle.gbm(W.gbm_key(0), 4096, **cfg)
    np.testing.assert_allclose(terminal[:4096].cpu().numpy(), head, rtol=1e-4)
    # E[S_T] = S0 exp(r T) under the risk-neutral measure
    assert abs(float(terminal.double().mean()) - cfg["s0"] * np.exp(cfg["r"] * cfg["t"])) < 0.02


def test_gray_scott_8192_fused_and_single_step_kernels_agree():
    import torch

    size = W.GRAY_SCOTT_CONFIG["size"]
    u0, v0 = W.gray_scott_initial_state(size)
    u, v = torch.from_numpy(u0).cuda(), torch.from_numpy(v0).cuda()
    steps = 18
    results = []
    for variant in (1, 2):
        with _native.thread_tuning(gs_variant=variant):
            call = H.gs_solver(size, size, call=pd.cuda_call_jit, math_mode=SAFE, steps=steps)
            results.append(call(u, v))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    # a window around a seeded patch corner equals the oracle run on the periodic sub-problem's light cone
    uo = results[1][0]
    assert torch.isfinite(uo).all() and float(uo.max()) <= 1.02 and float(results[1][1].min()) >= 0.0
    # splitting the run does not change it: 18 steps == 10 steps then 8 steps
    a = H.gs_solver(size, size, call=pd.cuda_call_jit, math_mode=SAFE, steps=10)(u, v)
    b = H.gs_solver(size, size, call=pd.cuda_call_jit, math_mode=SAFE, steps=8)(*a)
    assert torch.equal(b[0], results[1][0]) and torch.equal(b[1], results[1][1])
    # and a corner block equals the oracle on the whole grid's corresponding block (small grid, same seed pattern)
    small_u, small_v = W.gray_scott_initial_state(256)
    got = H.gs_solver(256, 256, call=pd.cuda_call_jit, math_mode=SAFE, steps=steps)(
        torch.from_numpy(small_u).cuda(), torch.from_numpy(small_v).cuda())
    want = oracle.gray_scott(small_u, small_v, steps=steps)
    np.testing.assert_array_equal(got[0].cpu().numpy(), want[0])


def test_kepler_one_million_orbits_100k_steps():
    """The df32 benchmark configuration, run as 100 launches of 1000 steps with
    the state resident on the device.  Error against float64 on a subset is
    the CPU df32 oracle's (the subset is bit-identical to it), and the energy
    drift of every orbit stays at the float64 integrator's level."""
    import torch

    cfg = W.KEPLER_CONFIG
    n, chunk = cfg["n"], 1000
    state64, pairs = W.kepler_ensemble(n)
    call = H.kepler_solver(n, call=pd.cuda_call_jit, dt=cfg["dt"], gm=cfg["gm"], steps=chunk)
    dev = [torch.from_numpy(p).cuda() for p in pairs]
    for _ in range(cfg["steps"] // chunk):
        dev = list(call(*dev))
    got = [d.cpu().numpy() for d in dev]
    sub = slice(0, 96)
    want = oracle.kepler_rk4_df32([p[sub] for p in pairs], dt=cfg["dt"], gm=cfg["gm"], steps=cfg["steps"])
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g[sub], w)
    truth = oracle.kepler_rk4_f64(state64[sub], dt=cfg["dt"], gm=cfg["gm"], steps=cfg["steps"])
    got64 = np.stack([W.join_df32(got[2 * i], got[2 * i + 1]) for i in range(4)], axis=1)
    err = np.hypot(got64[sub, 0] - truth[:, 0], got64[sub, 1] - truth[:, 1])
    f32 = oracle.kepler_rk4_f32(state64[sub].astype(np.float32), dt=cfg["dt"], gm=cfg["gm"], steps=cfg["steps"])
    err32 = np.hypot(f32[:, 0] - truth[:, 0], f32[:, 1] - truth[:, 1])
    assert err.max() < 1e-3 * err32.max()
    e0, e1 = W.kepler_energy(state64), W.kepler_energy(got64)
    drift = np.abs(e1 - e0) / np.abs(e0)
    drift_truth = np.abs(W.kepler_energy(truth) - e0[sub]) / np.abs(e0[sub])
    assert np.isfinite(got64).all()
    assert drift.max() < 10 * max(drift_truth.max(), 1e-12) + 1e-9
