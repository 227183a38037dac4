"""Generates the known-answer fixtures in this directory from the CPU oracle.

    python tests/golden/make_golden.py

Each .npz holds the seeded inputs and the oracle's outputs for one kernel
family at a size the oracle finishes in well under a second.  The RK4 fixture
additionally stores the output of the reference's own emitted kernel
(tests/golden/rk4_lotka_volterra.metal in the reference, compiled for the CPU
by oracle/build.py), which needs the reference checkout and is therefore
produced here, once, rather than on the GPU box.  RNG vectors are the oracle's
restatement of src/palladium/emit/rules.py:121-201; they are NOT vectors
published for Threefry or produced by JAX (not installed), so they guard
against drift, not against a shared misreading of the specification.
"""

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE))

import oracle  # noqa: E402
from palladium_b200 import workloads as W  # noqa: E402


def main():
    # ---- RK4 Lotka-Volterra: reference distributions and benchmark distributions
    rng = np.random.default_rng(17)
    n = 512
    ref_args = [rng.uniform(lo, hi, n).astype(np.float32)
                for lo, hi in ((0.8, 1.2), (0.8, 1.2), (0.9, 1.3), (0.3, 0.5), (0.08, 0.12), (0.3, 0.5))]
    gx, gy = oracle.lv_rk4_reference_golden(*ref_args)   # the reference's emitted kernel, 500 steps
    ox, oy = oracle.lv_rk4(*ref_args, dt=0.01, steps=500)
    assert np.array_equal(gx, ox) and np.array_equal(gy, oy)
    bench_args = W.lotka_volterra_ensemble(1000, seed=17)
    bx, by = oracle.lv_rk4(*bench_args, dt=0.01, steps=1000)
    np.savez_compressed(HERE / "lv_rk4.npz", ref_inputs=np.stack(ref_args), ref_golden_x=gx, ref_golden_y=gy,
                        bench_inputs=np.stack(bench_args), bench_x=bx, bench_y=by)

    # ---- Threefry
    key = np.array([0x12345678, 0x9ABCDEF0], np.uint32)
    data = np.array([0, 1, 17, 0xFFFFFFFF, 123456789], np.uint32)
    np.savez_compressed(HERE / "threefry.npz", key=key, bits=oracle.random_bits(key, 64),
                        uniform=oracle.uniform(key, 64), data=data, fold_in=oracle.fold_in(key, data),
                        fold_uniform=oracle.fold_uniform(key, 8, 4),
                        block=oracle.threefry2x32(key, np.array([7, 9], np.uint32)))

    # ---- adaptive BS3(2): benchmark tolerances, both pow flavours
    x0, v0, mu = W.van_der_pol_ensemble(64, seed=3)
    cfg = dict(t1=20.0, rtol=1e-6, atol=1e-8, dt0=1e-3, max_steps=100_000)
    pd_out = oracle.vdp_bs32(x0, v0, mu, pow="pd", **cfg)
    libm_out = oracle.vdp_bs32(x0, v0, mu, pow="libm", **cfg)
    np.savez_compressed(HERE / "vdp_bs32.npz", x0=x0, v0=v0, mu=mu, pd=np.stack(pd_out), libm=np.stack(libm_out))

    # ---- GBM
    gkey = W.gbm_key(0)
    cfg = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=252)
    terminal, payoff = oracle.gbm(gkey, 2048, **cfg)
    np.savez_compressed(HERE / "gbm.npz", key=gkey, terminal=terminal, payoff=payoff)

    # ---- Gray-Scott
    u0, v0g = W.gray_scott_initial_state(64, seed=11, patches=4, patch=16)
    u, v = oracle.gray_scott(u0, v0g, steps=100)
    np.savez_compressed(HERE / "gray_scott.npz", u0=u0, v0=v0g, u=u, v=v)

    # ---- df32
    lv_args = W.lotka_volterra_ensemble(256, seed=17)
    dx, dy = oracle.lv_rk4_df32(*lv_args, dt=0.01, steps=500)
    state64, pairs = W.kepler_ensemble(256, seed=5)
    kout = oracle.kepler_rk4_df32(pairs, dt=1e-3, steps=1000)
    truth = oracle.kepler_rk4_f64(state64, dt=1e-3, steps=1000)
    np.savez_compressed(HERE / "df32.npz", lv_inputs=np.stack(lv_args), lv_x=dx, lv_y=dy, kepler_pairs=np.stack(pairs),
                        kepler_out=np.stack(kout), kepler_truth=truth)
    reference_numpy_fixtures(lv_args)
    reference_threefry_fixture()
    reference_gbm_fixture()
    reference_kernel_fixture()
    reference_df32_fixture(lv_args)
    print("golden fixtures written to", HERE)


def _reference_function(path: Path, name: str, namespace: dict):
    """One function of a reference example, taken out of its module by name: the
    examples import JAX and the Metal runtime at the top, which are not installed,
    but these helpers are plain NumPy / SciPy."""
    import ast

    tree = ast.parse(path.read_text())
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
    code = compile(ast.Module(body=[node], type_ignores=[]), str(path), "exec")
    exec(code, namespace)
    return namespace[name]


def reference_threefry_fixture():
    """Outputs of the Threefry block exactly as the reference's emitter writes
    it (`_emit_threefry2x32`, src/palladium/emit/rules.py:121-165, run from the
    checkout and compiled as C by oracle/build.py), with the counter
    constructions of its random_bits and fold_in rules (:168-201)."""
    from oracle import build as oracle_build

    if oracle_build.build_reference_threefry() is None:
        print("reference checkout not found: threefry_reference.npz left as it is")
        return
    rng = np.random.default_rng(2024)
    keys = rng.integers(0, 2 ** 32, (16, 2), dtype=np.uint64).astype(np.uint32)
    keys[0] = (0, 0)
    keys[1] = (0xFFFFFFFF, 0xFFFFFFFF)
    counters = rng.integers(0, 2 ** 32, (16, 2), dtype=np.uint64).astype(np.uint32)
    counters[0] = (0, 0)
    counters[1] = (0xFFFFFFFF, 0xFFFFFFFF)
    blocks = np.stack([oracle.reference_threefry(k, c)[0] for k, c in zip(keys, counters)])
    data = np.array([0, 1, 2, 17, 251, 252, 0x7FFFFFFF, 0xFFFFFFFF], np.uint32)
    bits = np.stack([oracle.reference_random_bits(k, 257) for k in keys[:4]])
    folds = np.stack([oracle.reference_fold_in(k, data) for k in keys[:4]])
    np.savez_compressed(HERE / "threefry_reference.npz", keys=keys, counters=counters, blocks=blocks, data=data,
                        bits=bits, folds=folds)


def reference_gbm_fixture():
    """Payoffs of the reference's hand-written Monte Carlo kernel `gbm_paths`
    (the GBM_MSL text of examples/03_sde_montecarlo.py:34-70, compiled for the CPU
    by oracle/build.py) at the example's own constants (:30-32) and at the
    benchmark's, plus pcg_hash on its own."""
    from oracle import build as oracle_build

    if oracle_build.build_reference_gbm() is None:
        print("reference checkout not found: gbm_pcg_reference.npz left as it is")
        return
    example = dict(s0=100.0, strike=105.0, r=0.03, sigma=0.2, t=1.0, steps=256)
    bench = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=252)
    values = np.concatenate([np.arange(4096, dtype=np.uint32),
                             np.random.default_rng(7).integers(0, 2 ** 32, 4096, dtype=np.uint64).astype(np.uint32)])
    np.savez_compressed(HERE / "gbm_pcg_reference.npz", example_payoff=oracle.reference_gbm_paths(4096, **example),
                        bench_payoff=oracle.reference_gbm_paths(4096, **bench), hash_in=values,
                        hash_out=oracle.reference_pcg_hash(values))


def reference_kernel_fixture():
    """Outputs of the reference's own Pallas kernel functions -- `lv_kernel`
    (examples/01_ode_ensembles.py:72-91), `vdp_adaptive_kernel`
    (examples/02_adaptive_lockstep.py:69-171), `pallas_gbm_kernel`
    (examples/03_sde_montecarlo.py:97-119) and `gray_scott_kernel`
    (examples/04_reaction_diffusion.py:61-74) -- taken out of the examples by name
    and executed on NumPy stand-ins for the jax / pl names they use
    (tests/golden/pallas_numpy.py), at the examples' own constants."""
    from oracle.build import REFERENCE_ROOT

    import pallas_numpy as PN

    examples = REFERENCE_ROOT / "examples"
    if not (examples / "02_adaptive_lockstep.py").exists():
        print("reference checkout not found: reference_kernels.npz left as it is")
        return
    out = {}
    # fixed-step RK4 (the example's DT and STEPS, examples/01:15-16)
    n = 64
    lv_in = W.lotka_volterra_ensemble(n)
    kernel = PN.load_kernel(examples / "01_ode_ensembles.py", "lv_kernel", (n,), dict(DT=0.01, STEPS=500),
                            outer="palladium_solver")
    xo, yo = PN.Ref(PN.f32(np.zeros(n))), PN.Ref(PN.f32(np.zeros(n)))
    kernel(*[PN.Ref(PN.f32(a)) for a in lv_in], xo, yo)
    out.update(lv_in=np.stack(lv_in), lv_x=np.asarray(xo.array), lv_y=np.asarray(yo.array))
    # adaptive BS3(2) (constants of examples/02:26-32)
    n = 48
    x0, v0, mu = W.van_der_pol_ensemble(n)
    consts = dict(T1=10.0, DT0=0.01, MAX_STEPS=6000, RTOL=1e-5, ATOL=1e-7, ERROR_ORDER=3, SAFETY=0.9, FACTORMIN=0.2,
                  FACTORMAX=10.0, pcoeff=0.4, icoeff=0.3)
    kernel = PN.load_kernel(examples / "02_adaptive_lockstep.py", "vdp_adaptive_kernel", (n,), consts,
                            outer="palladium_solver")
    outs = [PN.Ref(PN.f32(np.zeros(n))) for _ in range(6)]
    kernel(PN.Ref(PN.f32(x0)), PN.Ref(PN.f32(v0)), PN.Ref(PN.f32(mu)), *outs)
    out.update(vdp_in=np.stack([x0, v0, mu]), vdp_out=np.stack([np.asarray(o.array) for o in outs]))
    # Monte Carlo with in-kernel Threefry (constants of examples/03:30-32)
    n = 512
    key = W.gbm_key(0)
    kernel = PN.load_kernel(examples / "03_sde_montecarlo.py", "pallas_gbm_kernel", (n,),
                            dict(T=1.0, N_STEPS=256, R=0.03, SIGMA=0.2, S0=100.0, K=105.0))
    payoff = PN.Ref(PN.f32(np.zeros(n)))
    kernel(PN.Ref(key), payoff)
    out.update(gbm_key=key, gbm_payoff=np.asarray(payoff.array))
    # stencil (constants of examples/04:36)
    n = 32
    u0, v0g = W.gray_scott_initial_state(n, seed=11, patches=2, patch=8)
    kernel = PN.load_kernel(examples / "04_reaction_diffusion.py", "gray_scott_kernel", (n, n),
                            dict(SIZE=n, DU=0.16, DV=0.08, F=0.035, KK=0.065, DT=1.0))
    u, v = PN.f32(u0.copy()), PN.f32(v0g.copy())
    for _ in range(25):
        uo, vo = PN.f32(np.zeros((n, n))), PN.f32(np.zeros((n, n)))
        kernel(PN.Ref(u), PN.Ref(v), PN.Ref(uo), PN.Ref(vo))
        u, v = uo, vo
    out.update(gs_u0=u0, gs_v0=v0g, gs_u=np.asarray(u), gs_v=np.asarray(v))
    # the five-output adaptive kernel of the reference's own test, on that test's own inputs:
    # tests/test_08_adaptive.py:33-142 (kernel), :157-171 (`_inputs`), the rng fixture of
    # tests/conftest.py:21-23 (seed 17); case (a) mild ensemble, case (b) 2 % stiff members
    test08 = REFERENCE_ROOT / "tests" / "test_08_adaptive.py"
    consts = dict(X0=2.0, V0=0.0, DT0=0.01, T1=10.0, MAX_STEPS=6000, RTOL=1e-5, ATOL=1e-7, pcoeff=0.4, icoeff=0.3,
                  error_order=3)
    n = 256
    kernel = PN.load_kernel(test08, "vdp_adaptive_kernel", (n,), consts)
    helpers = {"np": np, **consts}
    for name in ("_mu_ensemble", "_inputs"):
        node = PN.extract_function(test08, name)
        import ast

        exec(compile(ast.Module(body=[node], type_ignores=[]), str(test08), "exec"), helpers)
    rng = np.random.default_rng(seed=17)
    for tag, stiff in (("mild", 0.0), ("stiff", 0.02)):
        x0, v0, mu = helpers["_inputs"](rng, n, stiff_fraction=stiff)
        outs = [PN.Ref(PN.f32(np.zeros(n))) for _ in range(5)]
        kernel(PN.Ref(PN.f32(x0)), PN.Ref(PN.f32(v0)), PN.Ref(PN.f32(mu)), *outs)
        out[f"test08_{tag}_in"] = np.stack([x0, v0, mu])
        out[f"test08_{tag}_out"] = np.stack([np.asarray(o.array) for o in outs])
    np.savez_compressed(HERE / "reference_kernels.npz", **out)


def reference_df32_fixture(lv_args):
    """Outputs of the reference's hand-written df32 kernel text (DF32_KERNEL,
    examples/05_df32_precision.py:27-80) compiled for the CPU on the oracle's
    restatement of the external df32 prelude (oracle/build.py): pins the kernel's
    structure, not the prelude's arithmetic."""
    from oracle import build as oracle_build

    if oracle_build.build_reference_df32() is None:
        print("reference checkout not found: df32_reference.npz left as it is")
        return
    x, y = oracle.reference_lv_rk4_df32(*lv_args, dt=0.01, steps=500)
    np.savez_compressed(HERE / "df32_reference.npz", lv_inputs=np.stack(lv_args), x=x, y=y)


def reference_numpy_fixtures(lv_args):
    """Outputs of the reference's own NumPy helpers, run here where its checkout
    is: the float64 RK4 truth of examples/05_df32_precision.py:95-109 (its module
    constants DT = 0.01, STEPS = 500, :24) and the closed-form call price of
    examples/03_sde_montecarlo.py:73-76."""
    from oracle.build import REFERENCE_ROOT

    ex05 = REFERENCE_ROOT / "examples" / "05_df32_precision.py"
    ex03 = REFERENCE_ROOT / "examples" / "03_sde_montecarlo.py"
    if not ex05.exists() or not ex03.exists():
        print("reference checkout not found: reference_numpy.npz left as it is")
        return
    from scipy.stats import norm

    f64 = _reference_function(ex05, "float64_reference", {"np": np, "DT": 0.01, "STEPS": 500})
    x64, y64 = f64(*lv_args)
    bs = _reference_function(ex03, "black_scholes_call", {"np": np, "norm": norm})
    cases = np.array([(100.0, 105.0, 1.0, 0.03, 0.2), (100.0, 100.0, 1.0, 0.05, 0.2), (80.0, 100.0, 0.5, 0.01, 0.35),
                      (120.0, 100.0, 2.0, 0.0, 0.1)])
    prices = np.array([bs(*c) for c in cases])
    np.savez_compressed(HERE / "reference_numpy.npz", lv_inputs=np.stack(lv_args), lv_f64_x=x64, lv_f64_y=y64,
                        bs_cases=cases, bs_prices=prices)


if __name__ == "__main__":
    main()
