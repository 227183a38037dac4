"""The oracle itself: against the committed golden fixtures, against the
reference's own emitted RK4 kernel, against its second (NumPy) restatement, and
against properties the algorithms must have.  No GPU."""

from fractions import Fraction
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import oracle_np
from palladium_b200 import workloads as W

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    return np.load(GOLDEN / f"{name}.npz")


# ------------------------------------------------------------------ RK4
def test_rk4_matches_reference_golden_fixture():
    """The fixture stores what the reference's emitted kernel
    (tests/golden/rk4_lotka_volterra.metal) produced; the oracle must be
    bit-identical to it."""
    g = load("lv_rk4")
    x, y = oracle.lv_rk4(*g["ref_inputs"], dt=0.01, steps=500)
    np.testing.assert_array_equal(x, g["ref_golden_x"])
    np.testing.assert_array_equal(y, g["ref_golden_y"])


def test_rk4_matches_compiled_reference_kernel_when_built():
    if oracle.reference_lib() is None:
        pytest.skip("oracle/_ref/libmslref.so not built (needs the reference checkout)")
    args = W.lotka_volterra_ensemble(4097)
    gx, gy = oracle.lv_rk4_reference_golden(*args)
    ox, oy = oracle.lv_rk4(*args, dt=0.01, steps=500)
    np.testing.assert_array_equal(gx, ox)
    np.testing.assert_array_equal(gy, oy)


def test_rk4_numpy_restatement_agrees_bit_for_bit():
    args = W.lotka_volterra_ensemble(777)
    cx, cy = oracle.lv_rk4(*args, dt=0.01, steps=300)
    nx, ny = oracle_np.lv_rk4(*args, dt=0.01, steps=300)
    np.testing.assert_array_equal(cx, nx)
    np.testing.assert_array_equal(cy, ny)


def test_rk4_benchmark_fixture_and_float64_agreement():
    g = load("lv_rk4")
    x, y = oracle.lv_rk4(*g["bench_inputs"], dt=0.01, steps=1000)
    np.testing.assert_array_equal(x, g["bench_x"])
    tx, ty = oracle.lv_rk4_f64(*g["bench_inputs"], dt=0.01, steps=1000)
    np.testing.assert_allclose(x, tx, rtol=2e-4)
    np.testing.assert_allclose(y, ty, rtol=2e-4)


def test_rk4_is_fourth_order():
    args = W.lotka_volterra_ensemble(16)
    ref = oracle.lv_rk4_f64(*args, dt=0.0005, steps=4000)[0]
    e1 = np.abs(oracle.lv_rk4_f64(*args, dt=0.02, steps=100)[0] - ref).max()
    e2 = np.abs(oracle.lv_rk4_f64(*args, dt=0.01, steps=200)[0] - ref).max()
    assert 12 < e1 / e2 < 20


def test_rk4_empty_and_single():
    empty = [np.zeros(0, np.float32)] * 6
    x, y = oracle.lv_rk4(*empty, dt=0.01, steps=10)
    assert x.size == 0 and y.size == 0
    one = [np.array([v], np.float32) for v in (1.0, 1.0, 1.0, 0.4, 1.0, 3.0)]
    assert oracle.lv_rk4(*one, dt=0.01, steps=0)[0][0] == 1.0


# ------------------------------------------------------------------ Threefry
def test_threefry_fixture_and_numpy_agreement():
    g = load("threefry")
    key = g["key"]
    np.testing.assert_array_equal(oracle.random_bits(key, 64), g["bits"])
    np.testing.assert_array_equal(oracle.uniform(key, 64), g["uniform"])
    np.testing.assert_array_equal(oracle.fold_in(key, g["data"]), g["fold_in"])
    np.testing.assert_array_equal(oracle.fold_uniform(key, 8, 4), g["fold_uniform"])
    np.testing.assert_array_equal(oracle_np.random_bits(key, 64), g["bits"])
    np.testing.assert_array_equal(oracle_np.uniform(key, 64), g["uniform"])
    np.testing.assert_array_equal(oracle_np.fold_in(key, g["data"]), g["fold_in"])
    a, b = oracle_np.threefry2x32(key[0], key[1], np.uint32(7), np.uint32(9))
    np.testing.assert_array_equal(np.array([a, b], np.uint32).ravel(), g["block"])


def test_random_bits_is_a_counter_function():
    """bits[i] depends on (key, i) only, so a longer draw extends a shorter one
    (the property `random_bits` with a flat-index counter gives)."""
    key = W.gbm_key(5)
    np.testing.assert_array_equal(oracle.random_bits(key, 100)[:10], oracle.random_bits(key, 10))


def test_uniform_statistics():
    u = oracle.uniform(W.gbm_key(11), 1 << 20)
    assert 0.0 <= u.min() and u.max() < 1.0
    assert abs(u.mean() - 0.5) < 1e-3
    assert abs(u.var() - 1 / 12) < 1e-3
    counts, _ = np.histogram(u, bins=64, range=(0, 1))
    chi2 = ((counts - u.size / 64) ** 2 / (u.size / 64)).sum()
    assert chi2 < 120  # 63 degrees of freedom
    # low bits of the raw draws are balanced as well
    bits = oracle.random_bits(W.gbm_key(11), 1 << 18)
    ones = np.unpackbits(bits.view(np.uint8)).mean()
    assert abs(ones - 0.5) < 2e-3
    assert abs(np.corrcoef(u[:-1], u[1:])[0, 1]) < 5e-3


def test_fold_in_streams_differ():
    key = W.gbm_key(7)
    rows = oracle.fold_uniform(key, 8, 4)
    assert len({tuple(r) for r in rows}) == 8


# ------------------------------------------------------------------ adaptive
VDP_CFG = dict(t1=20.0, rtol=1e-6, atol=1e-8, dt0=1e-3, max_steps=100_000)


def test_vdp_fixture():
    g = load("vdp_bs32")
    for flavour in ("pd", "libm"):
        out = oracle.vdp_bs32(g["x0"], g["v0"], g["mu"], pow=flavour, **VDP_CFG)
        np.testing.assert_array_equal(np.stack(out), g[flavour])


def test_vdp_invariants():
    x0, v0, mu = W.van_der_pol_ensemble(128)
    t, x, v, steps, rejected, real = oracle.vdp_bs32(x0, v0, mu, pow="pd", **VDP_CFG)
    assert np.all(t == 20.0)                      # every trajectory lands exactly on T1
    np.testing.assert_array_equal(steps + rejected, VDP_CFG["max_steps"])  # accept or reject, every iteration
    assert np.all(real <= steps) and np.all(real > 0)
    assert np.std(real) > 0                      # adaptivity is per trajectory
    # the two pow flavours solve the same problem to the solver's tolerance
    other = oracle.vdp_bs32(x0, v0, mu, pow="libm", **VDP_CFG)
    np.testing.assert_allclose(x, other[1], rtol=2e-3, atol=2e-3)


def test_vdp_budget_exhaustion_is_reported_not_hidden():
    x0, v0, mu = W.van_der_pol_ensemble(8)
    t, *_rest, real = oracle.vdp_bs32(x0, v0, mu, pow="pd", **{**VDP_CFG, "max_steps": 50})
    assert np.all(t < 20.0) and np.all(real <= 50)


def test_vdp_reference_configuration_counts_are_stable_across_pow():
    """On the reference's mild ensemble and tolerances the step counts of the
    two pow flavours differ by a handful at most (its GPU-vs-CPU bar is 20,
    tests/test_08_adaptive.py:181-189)."""
    rng = np.random.default_rng(17)
    n = 256
    mu = rng.uniform(0.5, 2.0, n).astype(np.float32)
    x0, v0 = np.full(n, 2.0, np.float32), np.zeros(n, np.float32)
    a = oracle.vdp_bs32(x0, v0, mu, pow="pd")
    b = oracle.vdp_bs32(x0, v0, mu, pow="libm")
    np.testing.assert_allclose(a[5], b[5], rtol=0, atol=20)
    np.testing.assert_allclose(a[0], 10.0, atol=1e-4)


def test_controller_powers_accuracy_and_domain():
    """(1 / err) ** c for the step controller: float arithmetic only, within 8 ulp of
    double precision over the range the error norm takes; exactly 1 at err = 1 (the
    controller's initial state); pd_powf's rules outside the normal positive range."""
    rng = np.random.default_rng(4)
    err = np.exp(rng.uniform(np.log(1e-9), np.log(1e9), 400_000)).astype(np.float32)
    for c in (0.7 / 3, -0.4 / 3, 0.5, -0.25):
        got = oracle.pd_ctrl_pow(err, np.float32(c)).astype(np.float64)
        want = (1.0 / err.astype(np.float64)) ** np.float64(np.float32(c))
        ulp = np.abs(got - want) / want / 2.0 ** -24
        assert ulp.max() < 8.0 and ulp.mean() < 2.0
    assert oracle.pd_ctrl_pow(np.float32(1.0), np.float32(0.2333))[()] == 1.0
    special = oracle.pd_ctrl_pow(np.array([0.0, np.inf, np.nan, 1e-42], np.float32), np.float32(0.25))
    assert special[0] == np.inf and special[1] == 0.0 and np.isnan(special[2])
    assert special[3] == np.inf      # 1 / err overflows for a subnormal err, as the reference's own 1 / err_norm does


def test_pd_powf_accuracy_and_domain():
    rng = np.random.default_rng(1)
    x = np.exp(rng.uniform(np.log(1e-9), np.log(1e9), 200_000)).astype(np.float32)
    for y in (np.float32(0.7 / 3), np.float32(-0.4 / 3)):
        got = oracle.pd_powf(x, y).astype(np.float64)
        want = np.power(x.astype(np.float64), np.float64(y))
        ulp = np.spacing(want.astype(np.float32)).astype(np.float64)
        assert np.max(np.abs(got - want) / ulp) < 1.0
    sp = oracle.pd_powf(np.array([0, 0, np.inf, np.nan, 1, 4], np.float32), np.array([0.2, -0.2, 0.2, 0.2, 0, 0.5], np.float32))
    assert sp[0] == 0 and np.isinf(sp[1]) and np.isinf(sp[2]) and np.isnan(sp[3]) and sp[4] == 1 and sp[5] == 2


# ------------------------------------------------------------------ GBM
GBM_CFG = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=252)


def test_gbm_fixture_and_numpy_agreement():
    g = load("gbm")
    terminal, payoff = oracle.gbm(g["key"], 2048, **GBM_CFG)
    np.testing.assert_allclose(terminal, g["terminal"], rtol=1e-6)  # libm may differ in the last ulp across hosts
    np.testing.assert_array_equal(payoff, np.maximum(terminal - np.float32(100.0), np.float32(0.0)))
    nt, _ = oracle_np.gbm(g["key"], 512, **GBM_CFG)
    np.testing.assert_allclose(nt, terminal[:512], rtol=1e-5)


def test_gbm_black_scholes_within_5_sigma():
    _, payoff = oracle.gbm(W.gbm_key(0), 1 << 17, **GBM_CFG)
    disc = np.exp(-0.05)
    price = disc * payoff.mean()
    stderr = disc * payoff.std(ddof=1) / np.sqrt(payoff.size)
    assert abs(price - oracle.black_scholes_call(100.0, 100.0, 1.0, 0.05, 0.2)) < 5 * stderr


def test_gbm_path_offset_selects_global_streams():
    key = W.gbm_key(3)
    whole, _ = oracle.gbm(key, 256, **GBM_CFG)
    part, _ = oracle.gbm(key, 64, path_offset=128, **GBM_CFG)
    np.testing.assert_array_equal(part, whole[128:192])


def test_pcg_hash_restatements_agree_and_price_matches_black_scholes():
    np.testing.assert_array_equal(oracle.pcg_hash(50_000), oracle_np.pcg_hash(np.arange(50_000)))
    u = oracle_np.pcg_uniform01(np.arange(1 << 18))
    assert 0.0 < u.min() and u.max() <= 1.0 and abs(u.mean() - 0.5) < 2e-3
    cfg = dict(s0=100.0, strike=105.0, r=0.03, sigma=0.2, t=1.0, steps=256)  # examples/03_sde_montecarlo.py:30-32
    _, payoff = oracle.gbm_pcg(1 << 16, **cfg)
    disc = np.exp(-0.03)
    price, stderr = disc * payoff.mean(), disc * payoff.std(ddof=1) / np.sqrt(payoff.size)
    assert abs(price - oracle.black_scholes_call(100.0, 105.0, 1.0, 0.03, 0.2)) < 5 * stderr
    part, _ = oracle.gbm_pcg(64, path_offset=1000, **cfg)
    whole, _ = oracle.gbm_pcg(1064, **cfg)
    np.testing.assert_array_equal(part, whole[1000:])


# ------------------------------------------------------------------ Gray-Scott
def test_gray_scott_fixture_and_numpy_agreement():
    g = load("gray_scott")
    u, v = oracle.gray_scott(g["u0"], g["v0"], steps=100)
    np.testing.assert_array_equal(u, g["u"])
    np.testing.assert_array_equal(v, g["v"])
    nu, nv = oracle_np.gray_scott(g["u0"], g["v0"], steps=100)
    np.testing.assert_array_equal(nu, u)
    np.testing.assert_array_equal(nv, v)


def test_gray_scott_close_to_roll_laplacian_baseline():
    """The reference's CPU baseline sums the neighbours in another order
    (examples/04_reaction_diffusion.py:38-58); the two agree to rounding."""
    u, v = W.gray_scott_initial_state(48, patches=3, patch=8)
    a, b = u.copy(), v.copy()
    F, K, DU, DV = np.float32(0.035), np.float32(0.065), np.float32(0.16), np.float32(0.08)

    def lap(z):
        return np.roll(z, 1, 0) + np.roll(z, -1, 0) + np.roll(z, 1, 1) + np.roll(z, -1, 1) - np.float32(4.0) * z

    for _ in range(50):
        uvv = a * b * b
        a, b = a + (DU * lap(a) - uvv + F * (np.float32(1.0) - a)), b + (DV * lap(b) + uvv - (F + K) * b)
    ou, ov = oracle.gray_scott(u, v, steps=50)
    np.testing.assert_allclose(ou, a, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ov, b, rtol=1e-5, atol=1e-6)


def test_gray_scott_translation_invariance():
    """Periodic boundaries: shifting the input shifts the output, bit for bit."""
    u, v = W.gray_scott_initial_state(32, patches=2, patch=8)
    a = oracle.gray_scott(u, v, steps=10)
    b = oracle.gray_scott(np.roll(u, (5, 9), (0, 1)), np.roll(v, (5, 9), (0, 1)), steps=10)
    np.testing.assert_array_equal(np.roll(a[0], (5, 9), (0, 1)), b[0])
    np.testing.assert_array_equal(np.roll(a[1], (5, 9), (0, 1)), b[1])


def test_gray_scott_slab_restatement_matches_periodic():
    rows, cols, k = 40, 24, 3
    rng = np.random.default_rng(2)
    u = (1 - 0.5 * rng.random((rows, cols))).astype(np.float32)
    v = (0.25 * rng.random((rows, cols))).astype(np.float32)
    want = oracle.gray_scott(u, v, steps=k)
    idx = np.arange(10 - k, 30 + k) % rows
    su, sv = oracle_np.gray_scott_slab(u[idx], v[idx], steps=k, halo=k)
    np.testing.assert_array_equal(su[k:-k], want[0][10:30])
    np.testing.assert_array_equal(sv[k:-k], want[1][10:30])


# ------------------------------------------------------------------ df32
def _frac(x):
    return Fraction(float(x))


def test_error_free_transforms_are_exact():
    rng = np.random.default_rng(4)
    a = (rng.standard_normal(300) * 10.0 ** rng.integers(-6, 6, 300)).astype(np.float32)
    b = (rng.standard_normal(300) * 10.0 ** rng.integers(-6, 6, 300)).astype(np.float32)
    s, e = oracle.eft("two_sum", a, b)
    p, q = oracle.eft("two_prod", a, b)
    for i in range(a.size):
        assert _frac(s[i]) + _frac(e[i]) == _frac(a[i]) + _frac(b[i])
        assert _frac(p[i]) + _frac(q[i]) == _frac(a[i]) * _frac(b[i])


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "sqrt", "recip", "rsqrt"])
def test_df32_operations_reach_double_float_accuracy(op):
    rng = np.random.default_rng(6)
    a64 = rng.uniform(0.1, 10.0, 5000)
    b64 = rng.uniform(0.1, 10.0, 5000)
    if op == "sub":
        b64 = a64 * (1 + rng.uniform(-1e-3, 1e-3, 5000))  # cancellation
    ah, al = W.split_df32(a64)
    bh, bl = W.split_df32(b64)
    a_exact, b_exact = W.join_df32(ah, al), W.join_df32(bh, bl)
    oh, ol = oracle.df_op(op, ah, al, bh, bl)
    got = W.join_df32(oh, ol)
    want = {"add": a_exact + b_exact, "sub": a_exact - b_exact, "mul": a_exact * b_exact,
            "div": a_exact / b_exact, "sqrt": np.sqrt(a_exact), "recip": 1.0 / a_exact, "rsqrt": 1.0 / np.sqrt(a_exact)}[op]
    scale = np.maximum(np.abs(want), np.abs(a_exact) * 1e-3) if op == "sub" else np.abs(want)
    assert np.max(np.abs(got - want) / scale) < 2.0 ** -43
    assert np.all(np.abs(ol) <= np.spacing(np.abs(oh)))  # normalised pair


def test_df32_fixture_and_accuracy():
    g = load("df32")
    x, y = oracle.lv_rk4_df32(*g["lv_inputs"], dt=0.01, steps=500)
    np.testing.assert_array_equal(x, g["lv_x"])
    out = oracle.kepler_rk4_df32(list(g["kepler_pairs"]), dt=1e-3, steps=1000)
    np.testing.assert_array_equal(np.stack(out), g["kepler_out"])
    got = np.stack([W.join_df32(out[2 * i], out[2 * i + 1]) for i in range(4)], axis=1)
    err = np.abs(got - g["kepler_truth"]).max()
    assert err < 1e-9
    state32 = np.stack([W.join_df32(g["kepler_pairs"][2 * i], g["kepler_pairs"][2 * i + 1]) for i in range(4)], axis=1)
    f32 = oracle.kepler_rk4_f32(state32.astype(np.float32), dt=1e-3, steps=1000)
    assert err < 1e-3 * np.abs(f32 - g["kepler_truth"]).max()


def test_kepler_float64_conserves_energy():
    state, _ = W.kepler_ensemble(64)
    out = oracle.kepler_rk4_f64(state, dt=1e-3, steps=2000)
    e0, e1 = W.kepler_energy(state), W.kepler_energy(out)
    assert np.max(np.abs(e1 - e0) / np.abs(e0)) < 1e-7


def test_lv_df32_beats_float32_against_float64():
    args = W.lotka_volterra_ensemble(512)
    tx, ty = oracle.lv_rk4_f64(*args, dt=float(np.float32(0.01)), steps=500)
    dx, dy = oracle.lv_rk4_df32(*args, dt=0.01, steps=500)
    fx, fy = oracle.lv_rk4(*args, dt=0.01, steps=500)
    assert np.abs(dx - tx).max() < np.abs(fx - tx).max()  # examples/05_df32_precision.py:197


def test_float64_truth_and_closed_form_price_match_the_references_own_numpy_code():
    """tests/golden/reference_numpy.npz holds outputs of the reference's
    `float64_reference` (examples/05_df32_precision.py:95-109) and
    `black_scholes_call` (examples/03_sde_montecarlo.py:73-76), run from its
    checkout by tests/golden/make_golden.py."""
    g = np.load(GOLDEN / "reference_numpy.npz")
    x, y = oracle.lv_rk4_f64(*g["lv_inputs"], dt=0.01, steps=500)
    np.testing.assert_array_equal(x, g["lv_f64_x"])
    np.testing.assert_array_equal(y, g["lv_f64_y"])
    for case, price in zip(g["bs_cases"], g["bs_prices"]):
        assert abs(oracle.black_scholes_call(*case) - price) <= 1e-12 * price
    # the df32 kernel's reason to exist, against the reference's own truth (examples/05:197)
    dx, dy = oracle.lv_rk4_df32(*g["lv_inputs"], dt=0.01, steps=500)
    fx, fy = oracle.lv_rk4(*g["lv_inputs"], dt=0.01, steps=500)
    assert np.max(np.abs(dx - g["lv_f64_x"])) < np.max(np.abs(fx - g["lv_f64_x"]))
    assert np.max(np.abs(dy - g["lv_f64_y"])) < np.max(np.abs(fy - g["lv_f64_y"]))


def test_threefry_matches_the_statements_the_references_emitter_writes():
    """tests/golden/threefry_reference.npz was produced by running the reference's
    `_emit_threefry2x32` (src/palladium/emit/rules.py:121-165) where it lies and
    compiling the emitted statements as C (oracle/build.py); this pins the block,
    the random_bits counter (0, flat index) with xor fold, and fold_in."""
    g = load("threefry_reference")
    for key, ctr, want in zip(g["keys"], g["counters"], g["blocks"]):
        np.testing.assert_array_equal(oracle.threefry2x32(key, ctr), want)
        a, b = oracle_np.threefry2x32(key[0], key[1], ctr[0], ctr[1])
        assert (int(a), int(b)) == (int(want[0]), int(want[1]))
    for key, bits, folds in zip(g["keys"], g["bits"], g["folds"]):
        np.testing.assert_array_equal(oracle.random_bits(key, bits.size), bits)
        np.testing.assert_array_equal(oracle.fold_in(key, g["data"]), folds)
    if oracle.reference_threefry_lib() is not None:     # live, where the reference checkout is
        rng = np.random.default_rng(99)
        for _ in range(50):
            key = rng.integers(0, 2 ** 32, 2, dtype=np.uint64).astype(np.uint32)
            ctr = rng.integers(0, 2 ** 32, 2, dtype=np.uint64).astype(np.uint32)
            np.testing.assert_array_equal(oracle.threefry2x32(key, ctr), oracle.reference_threefry(key, ctr)[0])


def test_gbm_pcg_equals_the_references_hand_written_kernel():
    """tests/golden/gbm_pcg_reference.npz: payoffs of the reference's own `gbm_paths`
    MSL kernel (examples/03_sde_montecarlo.py:34-70) compiled for the CPU through
    oracle/msl_shim (oracle/build.py).  Same C library, same operation order:
    the restatement is bit-identical."""
    g = load("gbm_pcg_reference")
    np.testing.assert_array_equal(oracle.pcg_hash(4096), g["hash_out"][:4096])
    np.testing.assert_array_equal(oracle_np.pcg_hash(g["hash_in"]), g["hash_out"])
    example = dict(s0=100.0, strike=105.0, r=0.03, sigma=0.2, t=1.0, steps=256)
    bench = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=252)
    for cfg, want in ((example, g["example_payoff"]), (bench, g["bench_payoff"])):
        _, payoff = oracle.gbm_pcg(want.size, **cfg)
        np.testing.assert_array_equal(payoff, want)


def test_oracle_equals_the_references_own_kernel_functions():
    """tests/golden/reference_kernels.npz: the reference's Pallas kernel functions
    (examples/01:72-91, 02:69-171, 03:97-119, 04:61-74) executed on NumPy stand-ins
    for the jax / pl names they use (tests/golden/pallas_numpy.py), with the C
    library's pow / exp / log / cos.  The C oracle restates each of them and must
    agree bit for bit: state, time, and all three counters of the adaptive loop."""
    g = load("reference_kernels")
    x, y = oracle.lv_rk4(*g["lv_in"], dt=0.01, steps=500)
    np.testing.assert_array_equal(x, g["lv_x"])
    np.testing.assert_array_equal(y, g["lv_y"])
    got = oracle.vdp_bs32(*g["vdp_in"], pow="libm", t1=10.0, rtol=1e-5, atol=1e-7, dt0=0.01, max_steps=6000)
    for have, want, name in zip(got, g["vdp_out"], ("t", "x", "v", "steps", "rejected", "real")):
        np.testing.assert_array_equal(have, want, err_msg=name)
    assert g["vdp_out"][4].max() > 0 and np.std(g["vdp_out"][5]) > 0      # rejections happen, counts differ
    _, payoff = oracle.gbm(g["gbm_key"], g["gbm_payoff"].size, s0=100.0, strike=105.0, r=0.03, sigma=0.2, t=1.0,
                           steps=256)
    np.testing.assert_array_equal(payoff, g["gbm_payoff"])
    assert 0.2 < np.mean(g["gbm_payoff"] > 0) < 0.6
    u, v = oracle.gray_scott(g["gs_u0"], g["gs_v0"], steps=25)
    np.testing.assert_array_equal(u, g["gs_u"])
    np.testing.assert_array_equal(v, g["gs_v"])
    nu, nv = oracle_np.gray_scott(g["gs_u0"], g["gs_v0"], steps=25)
    np.testing.assert_array_equal(nu, g["gs_u"])
    np.testing.assert_array_equal(nv, g["gs_v"])


def test_df32_kernel_structure_equals_the_references_kernel_text():
    """tests/golden/df32_reference.npz: the reference's DF32_KERNEL text
    (examples/05_df32_precision.py:27-80) compiled for the CPU on the oracle's df32
    prelude.  Operation order, constants (0.5f * dt, dt / 6.0f in float32) and the
    RK4 combination are the reference's; the prelude arithmetic is restated."""
    g = load("df32_reference")
    x, y = oracle.lv_rk4_df32(*g["lv_inputs"], dt=0.01, steps=500)
    np.testing.assert_array_equal(x, g["x"])
    np.testing.assert_array_equal(y, g["y"])


def test_oracle_equals_the_references_test_kernel_on_its_own_inputs():
    """The five-output adaptive kernel of tests/test_08_adaptive.py:33-142 in the
    reference, run on that test's own inputs (`_inputs`, rng seed 17): the mild
    ensemble of its case (a) and the 2 % stiff ensemble of its case (b)."""
    g = load("reference_kernels")
    for tag in ("mild", "stiff"):
        got = oracle.vdp_bs32(*g[f"test08_{tag}_in"], pow="libm", t1=10.0, rtol=1e-5, atol=1e-7, dt0=0.01,
                              max_steps=6000)
        for have, want, name in zip(got[:5], g[f"test08_{tag}_out"], ("t", "x", "v", "steps", "rejected")):
            np.testing.assert_array_equal(have, want, err_msg=f"{tag} {name}")
    assert np.all(g["test08_stiff_out"][0] == 10.0) and g["test08_stiff_in"][2].max() > 300.0
