"""Timing of the kernel families other than the headline RK4 ensemble.

`quick_summary()` measures each family once at a reduced, stated size with the
inputs resident on the device (CUDA events on the launch stream) and returns a
dict that `bench.py` embeds in its JSON line under "families".
`run(...)` makes one family the benchmark's main workload
(`bench.py --workload vdp_bs32|gbm|gray_scott|kepler_df32`), one rank per GPU.

Algorithmic costs used for the roofline fractions:
  adaptive BS3(2): one attempt = 97 float operations + one log2, two exp2 and
      three divisions, which are not counted (from the kernel body; stall
      iterations are not attempts);
  GBM: one path-step = 4 Threefry-2x32-20 blocks = 4 x (20 rounds x 3 + 5 x 3 + 2)
      = 308 32-bit integer operations as written in the specification, plus
      log, sqrt, cos, exp;
  Gray-Scott: one cell-step = 16 bytes (read u, v; write u, v);
  df32: one trajectory-step counted from pd_math.h (see DF32_FLOPS).
"""

from __future__ import annotations

import json
import time

import numpy as np

VDP_FLOPS_PER_ATTEMPT = 97
GBM_INT_OPS_PER_PATH_STEP = 4 * (20 * 3 + 5 * 3 + 2)
GS_BYTES_PER_CELL_STEP = 16
# float operations per df32 primitive (pd_math.h), an FMA counted as 2: two_sum 6, fast_two_sum 3, two_prod 3
DF_ADD, DF_MUL = 6 + 6 + 1 + 3 + 1 + 3, 3 + 2 + 2 + 3
DF_DIV = 3 + 2 * (DF_MUL + DF_ADD) + 3 + DF_ADD
DF_SQRT = 1 + 3 + DF_ADD + 1 + 1 + 3
# LV: 4 rhs x (5 mul + 2 sub) + 3 advances x 2 x (mul + add) + combine 2 x (2 mul + 3 add) + final advance 2 x (mul + add)
DF32_LV_FLOPS = 4 * (5 * DF_MUL + 2 * DF_ADD) + 3 * 2 * (DF_MUL + DF_ADD) + 2 * (2 * DF_MUL + 3 * DF_ADD) + 2 * (DF_MUL + DF_ADD)
DF_RECIP = 1 + 3 + 2 + 2 + 1 + 3
# reciprocal square root: a/2, three float Newton steps of 4, two_prod, df_mul, residual 2, second-order term 3,
# correction 2, fast_two_sum 3 (the integer seed is not a float operation)
DF_RSQRT = 1 + 3 * 4 + 3 + DF_MUL + 2 + 3 + 2 + 3
# Kepler rhs: 2 mul + add, reciprocal square root, its cube (2 mul), 2 mul; GM = 1 costs nothing (negation is free)
_KEP_RHS = 2 * DF_MUL + DF_ADD + DF_RSQRT + 2 * DF_MUL + 2 * DF_MUL
# combine: two exact doublings (2 flops each) and three adds per component
DF32_KEPLER_FLOPS = 4 * _KEP_RHS + 3 * 4 * (DF_MUL + DF_ADD) + 4 * (2 * 2 + 3 * DF_ADD) + 4 * (DF_MUL + DF_ADD)
HBM_PEAK_FALLBACK_GBS = 6650.0


def _hbm_peak_gbs() -> tuple[float, str]:
    from pathlib import Path

    path = Path(__file__).resolve().parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "of measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return HBM_PEAK_FALLBACK_GBS, "of fallback (6.65 TB/s)"


def _time(fn, warmup: int, iters: int) -> float:
    """Average milliseconds per call of fn(), CUDA events on the current stream."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _shaped(shape, dtype=np.float32):
    from palladium_b200 import pl

    return pl.ShapeDtypeStruct(shape, dtype)


# ----------------------------------------------------------------------------- per family
def bench_vdp(n: int, math_mode="relaxed", warmup: int = 1, iters: int = 3, fma_peak: float | None = None) -> dict:
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    cfg = {k: v for k, v in W.VDP_CONFIG.items() if k not in ("n", "seed")}
    call = cuda_call_jit(families.vdp_bs32(**cfg), grid=(n,),
                         out_shape=(_shaped((n, 2)), _shaped((n,), np.int32), _shaped((n,), np.int32)),
                         math_mode=math_mode)
    dev = [torch.from_numpy(a).cuda() for a in W.van_der_pol_ensemble(n)]
    out = call(*dev)
    ms = _time(lambda: call(*dev), warmup, iters)
    accepted, rejected = out[1].double(), out[2].double()
    attempts = float((accepted + rejected).sum())
    res = {"workload": "adaptive BS3(2) Van der Pol", "trajectories": n, "math_mode": str(math_mode), "ms": ms,
           "attempts": attempts, "attempts_per_s": attempts / (ms * 1e-3),
           "mean_attempts": attempts / n, "max_attempts": float((accepted + rejected).max()),
           "mean_rejected": float(rejected.mean()), "trajectories_per_s": n / (ms * 1e-3)}
    if fma_peak:
        res["frac_of_fp32_peak"] = res["attempts_per_s"] * VDP_FLOPS_PER_ATTEMPT / fma_peak
    return res


VDP_RHS = "dy[0] = y[1];\ndy[1] = (p[0]*(1.0f - y[0]*y[0]))*y[1] - y[0];"


def bench_vdp_pair(n: int, method: str = "tsit5", math_mode="safe", warmup: int = 1, iters: int = 3) -> dict:
    """The Van der Pol configuration of `bench_vdp` (same ensemble, t1 and tolerances) through
    `custom_ode` with a seven-stage 5(4) pair: what the same job costs with the method the
    reference's CPU comparison integrates with."""
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    cfg = {k: v for k, v in W.VDP_CONFIG.items() if k not in ("n", "seed", "error_order")}
    call = cuda_call_jit(families.custom_ode(VDP_RHS, 2, 1, method=method, **cfg), grid=(n,),
                         out_shape=tuple(_shaped((n,)) for _ in range(6)), math_mode=math_mode)
    dev = [torch.from_numpy(a).cuda() for a in W.van_der_pol_ensemble(n)]
    out = call(*dev)
    ms = _time(lambda: call(*dev), warmup, iters)
    attempts = float((out[4].double() + out[5].double()).sum())
    return {"workload": f"adaptive {method} Van der Pol (custom_ode)", "trajectories": n, "math_mode": str(math_mode),
            "ms": ms, "attempts": attempts, "attempts_per_s": attempts / (ms * 1e-3), "mean_attempts": attempts / n,
            "all_reached_t1": bool((out[0] == cfg["t1"]).all()), "trajectories_per_s": n / (ms * 1e-3)}


def bench_gbm(n: int, math_mode="fast", warmup: int = 1, iters: int = 3, int_peak: float | None = None) -> dict:
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    cfg = {k: v for k, v in W.GBM_CONFIG.items() if k not in ("n", "seed")}
    call = cuda_call_jit(families.gbm_threefry(output="terminal", **cfg), grid=(n,),
                         out_shape=(_shaped((n,)), _shaped((2,), np.float64)), math_mode=math_mode)
    key = torch.from_numpy(W.gbm_key(0)).cuda()
    out, sums = call(key)
    ms = _time(lambda: call(key), warmup, iters)
    s1, s2 = (float(v) for v in sums.cpu())
    disc = float(np.exp(-cfg["r"] * cfg["t"]))
    mean = s1 / n
    stderr = disc * float(np.sqrt(max(s2 / n - mean * mean, 0.0) / n))
    path_steps = float(n) * cfg["steps"]
    res = {"workload": "GBM Monte Carlo, Threefry in-kernel", "paths": n, "steps": cfg["steps"],
           "math_mode": str(math_mode), "ms": ms, "path_steps_per_s": path_steps / (ms * 1e-3),
           "hashes_per_s": 4 * path_steps / (ms * 1e-3), "price": disc * mean, "stderr": stderr}
    from math import erf, exp, log, sqrt

    d1 = (log(cfg["s0"] / cfg["strike"]) + (cfg["r"] + cfg["sigma"] ** 2 / 2) * cfg["t"]) / (cfg["sigma"] * sqrt(cfg["t"]))
    d2 = d1 - cfg["sigma"] * sqrt(cfg["t"])
    cdf = lambda x: 0.5 * (1.0 + erf(x / sqrt(2.0)))  # noqa: E731
    exact = cfg["s0"] * cdf(d1) - cfg["strike"] * exp(-cfg["r"] * cfg["t"]) * cdf(d2)
    res["black_scholes"] = exact
    res["sigmas_from_black_scholes"] = abs(res["price"] - exact) / stderr if stderr else None
    if int_peak:
        res["frac_of_int32_peak"] = res["path_steps_per_s"] * GBM_INT_OPS_PER_PATH_STEP / int_peak
    return res


def bench_gbm_pcg(n: int, math_mode="fast", warmup: int = 1, iters: int = 3) -> dict:
    """The reference's hand-written variant (pcg_hash), at its own constants
    (examples/03_sde_montecarlo.py:30-32)."""
    from palladium_b200 import cuda_call_jit, families

    call = cuda_call_jit(families.gbm_pcg(), grid=(n,), out_shape=(_shaped((n,)), _shaped((2,), np.float64)),
                         math_mode=math_mode)
    out, sums = call.on_device()
    ms = _time(lambda: call.on_device(), warmup, iters)
    s1, s2 = (float(v) for v in sums.cpu())
    disc = float(np.exp(-0.03))
    mean = s1 / n
    return {"workload": "GBM Monte Carlo, pcg_hash (the reference's hand-written kernel)", "paths": n, "steps": 256,
            "math_mode": str(math_mode), "ms": ms, "path_steps_per_s": float(n) * 256 / (ms * 1e-3),
            "price": disc * mean, "stderr": disc * float(np.sqrt(max(s2 / n - mean * mean, 0.0) / n))}


def bench_gray_scott(size: int, steps: int, math_mode="fast", warmup: int = 1, iters: int = 3) -> dict:
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    cfg = {k: v for k, v in W.GRAY_SCOTT_CONFIG.items() if k not in ("steps", "size", "seed")}
    call = cuda_call_jit(families.gray_scott(steps=steps, **cfg), grid=(size, size),
                         out_shape=(_shaped((size, size)), _shaped((size, size))), math_mode=math_mode)
    u = torch.rand((size, size), device="cuda") * 0.5 + 0.5
    v = torch.rand((size, size), device="cuda") * 0.25
    ms = _time(lambda: call(u, v), warmup, iters)
    cell_steps = float(size) * size * steps
    peak, peak_note = _hbm_peak_gbs()
    gbs = cell_steps * GS_BYTES_PER_CELL_STEP / (ms * 1e-3) / 1e9
    return {"workload": "Gray-Scott periodic 5-point stencil", "size": size, "steps_per_call": steps,
            "math_mode": str(math_mode), "ms": ms, "ms_per_step": ms / steps,
            "cell_steps_per_s": cell_steps / (ms * 1e-3), "algorithmic_gbs": gbs, "hbm_peak_gbs": peak,
            "frac_of_hbm_peak": gbs / peak, "peak_note": peak_note, "frac_of_8tbs_nominal": gbs / 8000.0}


def bench_kepler(n: int, steps: int, warmup: int = 1, iters: int = 2, fma_peak: float | None = None) -> dict:
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    call = cuda_call_jit(families.kepler_rk4_df32(dt=W.KEPLER_CONFIG["dt"], gm=1.0, steps=steps), grid=(n,),
                         out_shape=tuple(_shaped((n,)) for _ in range(8)), math_mode="safe")
    _, pairs = W.kepler_ensemble(n)
    dev = [torch.from_numpy(a).cuda() for a in pairs]
    ms = _time(lambda: call(*dev), warmup, iters)
    ts = float(n) * steps
    res = {"workload": "df32 RK4 Kepler orbits", "trajectories": n, "steps_per_call": steps, "ms": ms,
           "trajectory_steps_per_s": ts / (ms * 1e-3), "flops_per_trajectory_step": DF32_KEPLER_FLOPS}
    if fma_peak:
        res["frac_of_fp32_peak"] = res["trajectory_steps_per_s"] * DF32_KEPLER_FLOPS / fma_peak
    return res


def bench_lv_df32(n: int, steps: int, warmup: int = 1, iters: int = 3, fma_peak: float | None = None) -> dict:
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    call = cuda_call_jit(families.lv_rk4_df32(0.01, steps), grid=(n,), out_shape=(_shaped((n,)), _shaped((n,))),
                         math_mode="safe")
    dev = [torch.from_numpy(a).cuda() for a in W.lotka_volterra_ensemble(n)]
    ms = _time(lambda: call(*dev), warmup, iters)
    ts = float(n) * steps
    res = {"workload": "df32 RK4 Lotka-Volterra", "trajectories": n, "steps_per_call": steps, "ms": ms,
           "trajectory_steps_per_s": ts / (ms * 1e-3), "flops_per_trajectory_step": DF32_LV_FLOPS}
    if fma_peak:
        res["frac_of_fp32_peak"] = res["trajectory_steps_per_s"] * DF32_LV_FLOPS / fma_peak
    return res


# The Lotka-Volterra right-hand side as a caller would hand it to `custom_ode`:
# in the reference's expression order, and factored so that each line is one
# multiply by a fused multiply-add.
CUSTOM_LV_TSIT5_MAX_STEPS = 64   # iterations of the adaptive loop: every trajectory of the benchmark ensembles ends within 48
LV_RHS = "dy[0] = p[0]*y[0] - (p[1]*y[0])*y[1];\ndy[1] = (p[2]*y[0])*y[1] - p[3]*y[1];"
CUSTOM_LV_RHS_FACTORED = "dy[0] = y[0]*fmaf(-p[1], y[1], p[0]);\ndy[1] = y[1]*fmaf(p[2], y[0], -p[3]);"


def bench_custom_ode(n: int, steps: int, math_mode: str = "fast", rhs: str = CUSTOM_LV_RHS_FACTORED, warmup: int = 2,
                     iters: int = 5, fma_peak: float | None = None) -> dict:
    """The run-time compiled RK4 kernel on the Lotka-Volterra system, beside the
    hand-written family on the same inputs."""
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    out_shape = (_shaped((n,)), _shaped((n,)))
    custom = cuda_call_jit(families.custom_ode(rhs, 2, 4, dt=0.01, steps=steps), grid=(n,), out_shape=out_shape,
                           math_mode=math_mode)
    family = cuda_call_jit(families.lv_rk4(0.01, steps), grid=(n,), out_shape=out_shape, math_mode=math_mode)
    dev = [torch.from_numpy(a).cuda() for a in W.lotka_volterra_ensemble(n)]
    ms = _time(lambda: custom(*dev), warmup, iters)
    ms_family = _time(lambda: family(*dev), warmup, iters)
    ts = float(n) * steps
    res = {"workload": "run-time compiled RK4 (custom_ode) on Lotka-Volterra", "trajectories": n,
           "steps_per_call": steps, "math_mode": math_mode, "ms": ms, "trajectory_steps_per_s": ts / (ms * 1e-3),
           "hand_written_family_ms": ms_family, "ratio_to_family": ms / ms_family}
    if fma_peak:
        res["frac_of_fp32_peak"] = res["trajectory_steps_per_s"] * 58 / fma_peak
    return res


LV_TSIT5_MAX_STEPS = 64   # iterations of the adaptive loop: every trajectory of the benchmark ensembles ends within 48
LV_RHS = "dy[0] = p[0]*y[0] - (p[1]*y[0])*y[1];\ndy[1] = (p[2]*y[0])*y[1] - p[3]*y[1];"


def reference_benchmark_ensemble(n: int, seed: int = 17):
    """The ensemble of the reference's benchmark suite (benchmarks/bench_ensembles.py:29-38): its
    ranges and draw order, not those of the named throughput configuration."""
    rng = np.random.default_rng(seed)
    ranges = ((0.8, 1.2), (0.8, 1.2), (0.9, 1.3), (0.3, 0.5), (0.08, 0.12), (0.3, 0.5))
    return tuple(rng.uniform(lo, hi, n).astype(np.float32) for lo, hi in ranges)


def bench_ensembles(repeats: int = 30) -> dict:
    """The reference's own benchmark definitions (benchmarks/bench_ensembles.py:24-26,78-118):
    the Lotka-Volterra ensemble at n = 10 000 and 100 000, dt 0.01, 500 steps, wall-clock ms of the
    eager call on host arrays with everything compiled beforehand (`bench_lv_palladium`); and its
    CPU comparison's job -- Tsit5 to t = 5 at rtol 1e-6, atol 1e-8 (`bench_lv_diffrax`) -- through
    `custom_ode(method="tsit5")` on the GPU.  The reference commits no results of either."""
    from palladium_b200 import cuda_call, families, pl

    spec_1 = pl.BlockSpec((1,), lambda i: (i,))
    out = {"definition": "benchmarks/bench_ensembles.py: dt 0.01, 500 steps, wall-clock ms per solve, medians"}
    for n in (10_000, 100_000):
        args = reference_benchmark_ensemble(n)
        rk4 = cuda_call(families.lv_rk4(0.01, 500), grid=(n,), in_specs=[spec_1] * 6, out_specs=(spec_1, spec_1),
                        out_shape=(_shaped((n,)), _shaped((n,))), math_mode="fast")
        tsit5 = cuda_call(families.custom_ode(LV_RHS, 2, 4, method="tsit5", t1=5.0, rtol=1e-6, atol=1e-8, dt0=0.01,
                                              max_steps=LV_TSIT5_MAX_STEPS),
                          grid=(n,), in_specs=[spec_1] * 6, out_specs=(spec_1,) * 6,
                          out_shape=tuple(_shaped((n,)) for _ in range(6)), math_mode="fast")

        def median_ms(call):
            call(*args)
            samples = []
            for _ in range(repeats):
                t0 = time.perf_counter()
                res = call(*args)
                samples.append(time.perf_counter() - t0)
            return float(np.median(samples)) * 1e3, res

        ms_rk4, _ = median_ms(rk4)
        ms_t5, res = median_ms(tsit5)
        out[f"n={n}"] = {"rk4_500_steps_eager_ms": ms_rk4, "tsit5_rtol1e-6_eager_ms": ms_t5,
                         "tsit5_accepted_steps_mean": float(res[5].mean()), "tsit5_all_reached_t1": bool((res[0] == 5.0).all())}
    return out


def fixed_costs(calls: int = 300) -> dict:
    """The per-call costs the reference documents for its runtime (docs/performance.md:35-48: a
    blocking dispatch floor of about 136 us, about 33 us per dispatch at in-flight depth 16, about
    0.25 ms of jit-path overhead at 16 KB and 1 MB buffers), measured the same way here: a kernel
    too small to matter (Lotka-Volterra, one RK4 step), medians of `calls` wall-clock samples."""
    import torch

    from palladium_b200 import cuda_call, cuda_call_jit, families, pl

    spec_1 = pl.BlockSpec((1,), lambda i: (i,))

    def make(n, jit):
        fam = families.lv_rk4(0.01, 1)
        if jit:
            return cuda_call_jit(fam, grid=(n,), out_shape=(_shaped((n,)), _shaped((n,))), math_mode="fast")
        return cuda_call(fam, grid=(n,), in_specs=[spec_1] * 6, out_specs=(spec_1, spec_1),
                         out_shape=(_shaped((n,)), _shaped((n,))), math_mode="fast")

    def median_us(fn, per=1):
        fn()
        samples = []
        for _ in range(calls):
            t0 = time.perf_counter()
            fn()
            samples.append((time.perf_counter() - t0) / per)
        return float(np.median(samples)) * 1e6

    out = {}
    for label, n in (("16KB", 4096), ("1MB", 262144)):
        arrays = [np.full(n, 1.0, np.float32) for _ in range(6)]
        eager, jit = make(n, False), make(n, True)
        dev = [torch.from_numpy(a).cuda() for a in arrays]
        outs = [torch.empty(n, device="cuda") for _ in range(2)]
        out[f"eager_blocking_call_us_{label}"] = median_us(lambda: eager(*arrays))
        out[f"jit_host_arrays_call_us_{label}"] = median_us(lambda: jit(*arrays))
        pinned = eager.pin(*arrays)
        out[f"pinned_inputs_call_us_{label}"] = median_us(pinned)

        def burst():
            pending = [eager.launch(*arrays) for _ in range(16)]
            for h in pending:
                h.wait()

        out[f"launch_wait_depth16_us_per_dispatch_{label}"] = median_us(burst, per=16)

        def stream_ordered():
            for _ in range(16):
                jit.on_device(*dev, out=outs)
            torch.cuda.synchronize()

        out[f"jit_device_tensors_us_per_call_depth16_{label}"] = median_us(stream_ordered, per=16)

        def blocking_device():
            jit(*dev)
            torch.cuda.synchronize()

        out[f"jit_device_tensors_blocking_call_us_{label}"] = median_us(blocking_device)
    out["reference_published"] = {"blocking_dispatch_floor_us": 136, "depth16_us_per_dispatch": 33,
                                  "jit_overhead_us_16KB": 190, "jit_overhead_us_1MB": 250,
                                  "hardware": "Apple M1 Pro (docs/performance.md:35-44)"}
    return out


def quick_summary(named: bool = True) -> dict:
    """Each family once at a reduced size that finishes in a few seconds, the headline kernel under the
    other two math modes, and (named=True) every benchmark configuration at its full named size."""
    from palladium_b200 import _native

    fma_peak = _native.measure_fp32_fma_peak()
    int_peak = _native.measure_int32_alu_peak()
    out = {"fp32_fma_peak_tflops": fma_peak / 1e12, "int32_alu_peak_tops": int_peak / 1e12}
    out["vdp_bs32"] = bench_vdp(1 << 18, "relaxed", fma_peak=fma_peak)
    out["vdp_bs32_safe"] = bench_vdp(1 << 18, "safe", fma_peak=fma_peak)
    out["gbm"] = bench_gbm(1 << 22, "fast", int_peak=int_peak)
    out["gbm_pcg"] = bench_gbm_pcg(1 << 22, "fast")
    out["gray_scott"] = bench_gray_scott(8192, 40, "fast")
    out["kepler_df32"] = bench_kepler(1 << 20, 100, fma_peak=fma_peak)
    out["lv_df32"] = bench_lv_df32(1 << 20, 100, fma_peak=fma_peak)
    out["custom_ode_lv"] = bench_custom_ode(1 << 22, 1000, "fast", fma_peak=fma_peak)
    out["vdp_tsit5_safe"] = bench_vdp_pair(1 << 18, "tsit5", "safe")
    out["fixed_costs"] = fixed_costs()
    out["bench_ensembles"] = bench_ensembles()
    out.update(named_rk4_modes(fma_peak))
    if named:
        out.update(named_configs(fma_peak, int_peak))
    return out


def full_configs(fma_peak: float, int_peak: float) -> dict:
    """Each benchmark configuration once at its full size on one GPU
    (`bench.py --workload full`): wall time of the whole job on the device."""
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    out = {"metric": "full_configurations", "value": None, "unit": "s", "scaling": "weak", "ms_per_step": None,
           "config": {"workload": "every benchmark configuration at full size, one GPU"}}
    r = bench_vdp(W.VDP_CONFIG["n"], "relaxed", warmup=1, iters=1, fma_peak=fma_peak)
    out["vdp_bs32_relaxed_1M"] = {"seconds": r["ms"] / 1e3, "attempts_per_s": r["attempts_per_s"]}
    r = bench_vdp(W.VDP_CONFIG["n"], "safe", warmup=1, iters=1, fma_peak=fma_peak)
    out["vdp_bs32_safe_1M"] = {"seconds": r["ms"] / 1e3, "attempts_per_s": r["attempts_per_s"]}
    r = bench_gbm(W.GBM_CONFIG["n"], "fast", warmup=1, iters=1, int_peak=int_peak)
    out["gbm_2^26"] = {"seconds": r["ms"] / 1e3, "path_steps_per_s": r["path_steps_per_s"], "price": r["price"],
                       "stderr": r["stderr"], "black_scholes": r["black_scholes"]}
    r = bench_gray_scott(W.GRAY_SCOTT_CONFIG["size"], W.GRAY_SCOTT_CONFIG["steps"], "fast", warmup=0, iters=1)
    out["gray_scott_8192_10000_steps"] = {"seconds": r["ms"] / 1e3, "us_per_step": r["ms_per_step"] * 1e3,
                                          "algorithmic_gbs": r["algorithmic_gbs"]}
    cfg = W.KEPLER_CONFIG
    n, chunk = cfg["n"], 1000
    call = cuda_call_jit(families.kepler_rk4_df32(dt=cfg["dt"], gm=cfg["gm"], steps=chunk), grid=(n,),
                         out_shape=tuple(_shaped((n,)) for _ in range(8)), math_mode="safe")
    _, pairs = W.kepler_ensemble(n)
    dev = [torch.from_numpy(a).cuda() for a in pairs]
    dev = list(call(*dev))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(cfg["steps"] // chunk):
        dev = list(call(*dev))
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3
    out["kepler_df32_1M_100000_steps"] = {"seconds": sec, "trajectory_steps_per_s": float(n) * cfg["steps"] / sec,
                                          "launches": cfg["steps"] // chunk}
    return out


# ----------------------------------------------------------------------------- the named configurations
# float64 RK4 of the two-body problem, one thread per orbit: the truth the df32
# result is measured against (examples/05_df32_precision.py:95-109 does the same
# for its system in NumPy).  A caller-written kernel, compiled at run time.
KEPLER_F64_SOURCE = r"""
struct S4 { double x, y, vx, vy; };
__device__ __forceinline__ S4 kep_f(S4 s, double gm) {
    const double r2 = s.x * s.x + s.y * s.y;
    const double w = gm / (r2 * sqrt(r2));
    S4 k; k.x = s.vx; k.y = s.vy; k.vx = -s.x * w; k.vy = -s.y * w; return k;
}
__device__ __forceinline__ S4 kep_adv(S4 s, S4 k, double h) {
    S4 r; r.x = s.x + h * k.x; r.y = s.y + h * k.y; r.vx = s.vx + h * k.vx; r.vy = s.vy + h * k.vy; return r;
}
extern "C" __global__ void kepler_rk4_f64(const double* state, const double* c, double* out,
                                          long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    const double dt = c[0], gm = c[1];
    const long long steps = (long long)c[2];
    S4 s; s.x = state[4 * i]; s.y = state[4 * i + 1]; s.vx = state[4 * i + 2]; s.vy = state[4 * i + 3];
    for (long long it = 0; it < steps; ++it) {
        const S4 k1 = kep_f(s, gm);
        const S4 k2 = kep_f(kep_adv(s, k1, 0.5 * dt), gm);
        const S4 k3 = kep_f(kep_adv(s, k2, 0.5 * dt), gm);
        const S4 k4 = kep_f(kep_adv(s, k3, dt), gm);
        S4 sum;
        sum.x = k1.x + 2.0 * k2.x + 2.0 * k3.x + k4.x;    sum.y = k1.y + 2.0 * k2.y + 2.0 * k3.y + k4.y;
        sum.vx = k1.vx + 2.0 * k2.vx + 2.0 * k3.vx + k4.vx; sum.vy = k1.vy + 2.0 * k2.vy + 2.0 * k3.vy + k4.vy;
        s = kep_adv(s, sum, dt / 6.0);
    }
    out[4 * i] = s.x; out[4 * i + 1] = s.y; out[4 * i + 2] = s.vx; out[4 * i + 3] = s.vy;
}
"""


def _wall(fn) -> float:
    import torch

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    fn()
    torch.cuda.synchronize()
    return time.perf_counter() - t0


def named_rk4_modes(fma_peak: float, n: int = 1 << 22, steps: int = 1000) -> dict:
    """The headline kernel under SAFE and RELAXED beside the timed FAST mode."""
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    dev = [torch.from_numpy(a).cuda() for a in W.lotka_volterra_ensemble(n)]
    out = {}
    for mode, parity in (("safe", "bit-exact against the oracle"),
                         ("relaxed", ">= 95 % of states within rtol 1e-5 of the oracle, all within 1e-4")):
        call = cuda_call_jit(families.lv_rk4(0.01, steps), grid=(n,), out_shape=(_shaped((n,)), _shaped((n,))),
                             math_mode=mode)
        ms = _time(lambda: call(*dev), 2, 5)
        out[f"rk4_lv_{mode}"] = {"trajectories": n, "rk4_steps": steps, "math_mode": mode, "ms": ms,
                                 "trajectory_steps_per_s": float(n) * steps / (ms * 1e-3),
                                 "frac_of_fp32_peak": float(n) * steps * 58 / (ms * 1e-3) / fma_peak, "parity": parity}
    return out


def named_configs(fma_peak: float, int_peak: float) -> dict:
    """Every other benchmark configuration at its full named size on one GPU:
    device-resident time, roofline fraction and the same job end to end from
    host arrays (upload, run, download inside the timed region)."""
    import torch

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    out = {}
    # ---- adaptive BS3(2), 1 000 000 Van der Pol oscillators -------------------------------------
    cfg = {k: v for k, v in W.VDP_CONFIG.items() if k not in ("n", "seed")}
    n = W.VDP_CONFIG["n"]
    host = W.van_der_pol_ensemble(n)
    pinned = [torch.from_numpy(a).pin_memory().numpy() for a in host]
    for mode in ("safe", "relaxed"):
        r = bench_vdp(n, mode, warmup=1, iters=2, fma_peak=fma_peak)
        call = cuda_call_jit(families.vdp_bs32(**cfg), grid=(n,),
                             out_shape=(_shaped((n, 2)), _shaped((n,), np.int32), _shaped((n,), np.int32)),
                             math_mode=mode)
        call(*pinned)
        sec = _wall(lambda: call(*pinned))
        r["e2e"] = {"seconds": sec, "attempts_per_s": r["attempts"] / sec, "h2d_bytes": 12 * n, "d2h_bytes": 16 * n,
                    "path": "cuda_call_jit(host arrays) -> pd_dispatch_host"}
        out[f"vdp_named_{mode}"] = r
    # ---- GBM, 2^26 paths ------------------------------------------------------------------------
    n = W.GBM_CONFIG["n"]
    r = bench_gbm(n, "fast", warmup=1, iters=2, int_peak=int_peak)
    gcfg = {k: v for k, v in W.GBM_CONFIG.items() if k not in ("n", "seed")}
    call = cuda_call_jit(families.gbm_threefry(output="terminal", **gcfg), grid=(n,),
                         out_shape=(_shaped((n,)), _shaped((2,), np.float64)), math_mode="fast")
    key = W.gbm_key(0)
    call(key)
    sec = _wall(lambda: call(key))
    r["e2e"] = {"seconds": sec, "path_steps_per_s": float(n) * gcfg["steps"] / sec, "h2d_bytes": 8,
                "d2h_bytes": 4 * n + 16, "path": "cuda_call_jit(host key) -> pd_dispatch_host, per-path prices downloaded"}
    out["gbm_named"] = r
    # ---- Gray-Scott 8192^2, 10 000 steps ---------------------------------------------------------
    size, steps = W.GRAY_SCOTT_CONFIG["size"], W.GRAY_SCOTT_CONFIG["steps"]
    gs = {k: v_ for k, v_ in W.GRAY_SCOTT_CONFIG.items() if k not in ("steps", "size", "seed")}
    call = cuda_call_jit(families.gray_scott(steps=steps, **gs), grid=(size, size),
                         out_shape=(_shaped((size, size)), _shaped((size, size))), math_mode="fast")
    u0, v0 = W.gray_scott_initial_state(size)
    hu, hv = torch.from_numpy(u0).pin_memory(), torch.from_numpy(v0).pin_memory()
    res = {}

    out_u, out_v = torch.empty_like(hu).pin_memory(), torch.empty_like(hv).pin_memory()   # page-locked, like the inputs

    def job():
        u, v = hu.cuda(non_blocking=True), hv.cuda(non_blocking=True)
        uo, vo = call(u, v)
        out_u.copy_(uo, non_blocking=True)
        out_v.copy_(vo, non_blocking=True)
        torch.cuda.synchronize()
        res["u"], res["v"] = out_u, out_v

    u, v = hu.cuda(), hv.cuda()
    warm = cuda_call_jit(families.gray_scott(steps=8, **gs), grid=(size, size),
                         out_shape=(_shaped((size, size)), _shaped((size, size))), math_mode="fast")
    warm(u, v)                       # same grid: kernel attributes set and the ping-pong scratch allocated
    ms = _time(lambda: call(u, v), 0, 1)
    e2e_sec = _wall(job)
    peak, note = _hbm_peak_gbs()
    cell_steps = float(size) * size * steps
    gbs = cell_steps * GS_BYTES_PER_CELL_STEP / (ms * 1e-3) / 1e9
    ru = res["u"]
    out["gray_scott_named"] = {
        "workload": "Gray-Scott 8192 x 8192 periodic, 10 000 steps, 64 seeded patches + noise", "size": size, "steps": steps,
        "math_mode": "fast", "seconds": ms / 1e3, "us_per_step": ms * 1e3 / steps,
        "cell_steps_per_s": cell_steps / (ms * 1e-3), "algorithmic_gbs": gbs, "frac_of_hbm_peak": gbs / peak,
        "peak_note": note, "launches": "one pd_launch call issues every fused launch back to back on the stream",
        "u_min": float(ru.min()), "u_max": float(ru.max()), "v_max": float(res["v"].max()),
        "finite": bool(torch.isfinite(ru).all()),
        "e2e": {"seconds": e2e_sec, "cell_steps_per_s": cell_steps / e2e_sec, "h2d_bytes": 8 * size * size,
                "d2h_bytes": 8 * size * size, "path": "pinned host fields uploaded, cuda_call_jit on device tensors, fields downloaded into pinned host memory"}}
    del u, v, res, ru
    # ---- df32 Kepler, 1 000 000 orbits x 100 000 steps --------------------------------------------
    kc = W.KEPLER_CONFIG
    n, chunk = kc["n"], 1000
    state64, pairs = W.kepler_ensemble(n)
    call = cuda_call_jit(families.kepler_rk4_df32(dt=kc["dt"], gm=kc["gm"], steps=chunk), grid=(n,),
                         out_shape=tuple(_shaped((n,)) for _ in range(8)), math_mode="safe")
    pinned = [torch.from_numpy(a).pin_memory() for a in pairs]
    got = {}

    def kepler_job():
        dev = [t.cuda(non_blocking=True) for t in pinned]
        for _ in range(kc["steps"] // chunk):
            dev = list(call(*dev))
        got["pairs"] = [d.cpu().numpy() for d in dev]

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev = [t.cuda() for t in pinned]
    dev = list(call(*dev))          # warm-up launch (1000 steps), not part of the job
    torch.cuda.synchronize()
    dev = [t.cuda() for t in pinned]
    e0.record()
    for _ in range(kc["steps"] // chunk):
        dev = list(call(*dev))
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3
    del dev
    e2e_sec = _wall(kepler_job)
    got64 = np.stack([W.join_df32(got["pairs"][2 * i], got["pairs"][2 * i + 1]) for i in range(4)], axis=1)
    # float64 truth on a subset of the same orbits, computed on the GPU by a caller-written kernel
    m = 1 << 14
    truth_call = cuda_call_jit(families.source_kernel(KEPLER_F64_SOURCE, "kepler_rk4_f64"), grid=(m,),
                               out_shape=_shaped((m, 4), np.float64), math_mode="safe")
    consts = torch.tensor([kc["dt"], kc["gm"], float(kc["steps"])], dtype=torch.float64, device="cuda")
    truth = truth_call(torch.from_numpy(np.ascontiguousarray(state64[:m])).cuda(), consts).cpu().numpy()
    err = np.hypot(got64[:m, 0] - truth[:, 0], got64[:m, 1] - truth[:, 1])
    e_start, e_end = W.kepler_energy(state64), W.kepler_energy(got64)
    drift = np.abs(e_end - e_start) / np.abs(e_start)
    drift_truth = np.abs(W.kepler_energy(truth) - e_start[:m]) / np.abs(e_start[:m])
    ts = float(n) * kc["steps"]
    out["kepler_named"] = {
        "workload": "df32 RK4 Kepler orbits, SAFE", "trajectories": n, "steps": kc["steps"], "launches": kc["steps"] // chunk,
        "seconds": sec, "trajectory_steps_per_s": ts / sec, "flops_per_trajectory_step": DF32_KEPLER_FLOPS,
        "frac_of_fp32_peak": ts * DF32_KEPLER_FLOPS / sec / fma_peak,
        "final_position_error_vs_float64": {"subset": m, "max": float(err.max()), "median": float(np.median(err)),
                                            "truth": "float64 RK4 of the same orbits, a run-time compiled kernel on the GPU"},
        "relative_energy_drift": {"max_all_orbits": float(drift.max()), "median_all_orbits": float(np.median(drift)),
                                  "max_float64_truth_subset": float(drift_truth.max())},
        "e2e": {"seconds": e2e_sec, "trajectory_steps_per_s": ts / e2e_sec, "h2d_bytes": 32 * n, "d2h_bytes": 32 * n,
                "path": "pinned host state uploaded, 100 cuda_call_jit launches on device tensors, state downloaded"}}
    return out


# ----------------------------------------------------------------------------- several GPUs
def _black_scholes(cfg: dict) -> float:
    from math import erf, exp, log, sqrt

    d1 = (log(cfg["s0"] / cfg["strike"]) + (cfg["r"] + cfg["sigma"] ** 2 / 2) * cfg["t"]) / (cfg["sigma"] * sqrt(cfg["t"]))
    d2 = d1 - cfg["sigma"] * sqrt(cfg["t"])
    cdf = lambda x: 0.5 * (1.0 + erf(x / sqrt(2.0)))  # noqa: E731
    return cfg["s0"] * cdf(d1) - cfg["strike"] * exp(-cfg["r"] * cfg["t"]) * cdf(d2)


def _gather_rows(local, world: int):
    """All ranks' equally sized first-axis shares, concatenated in rank order (on every rank)."""
    import torch
    import torch.distributed as dist

    full = torch.empty((local.shape[0] * world, *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(full, local.contiguous())
    return full


def multi_gpu_gbm(rank: int, world: int, barrier, max_over_ranks, math_mode: str = "fast", paths_per_gpu: int = 1 << 24,
                  iters: int = 3) -> dict:
    """The Monte Carlo on `world` GPUs: path slabs keyed by global path index, one
    all-reduce of two float64 sums per pass (examples/03_sde_montecarlo.py:137-146
    prices from one device's payoffs).  Checked in the same run: a 2^20-path case
    priced by all ranks together against rank 0 pricing it alone."""
    import torch

    from palladium_b200 import _native, sharded
    from palladium_b200 import workloads as W

    cfg = {k: v for k, v in W.GBM_CONFIG.items() if k not in ("n", "seed")}
    key = W.gbm_key(0)
    # ---- the check: every rank's paths and the all-reduced sums against one rank alone ----
    n_check = 1 << 20
    together = sharded.gbm_monte_carlo(key, n_check, cfg, math_mode=math_mode)
    everyone = _gather_rows(together.local_output, world) if n_check % world == 0 else None
    check = None
    if rank == 0:
        alone_out, alone_sums = sharded._cuda_gbm_paths(key, 0, n_check, cfg, math_mode, "terminal")
        a1, a2 = (float(x) for x in alone_sums.cpu())
        check = {
            "paths": n_check,
            # payoffs are multiples of 2^-17 (s >= strike = 100), so their float64 sum is exact in any order
            "sum_payoff_equal_single_rank": together.sums[0] == a1,
            "sum_payoff_sq_rel_diff": abs(together.sums[1] - a2) / a2 if a2 else 0.0,
            "per_path_outputs_equal_single_rank": bool(torch.equal(everyone, alone_out)) if everyone is not None else None,
        }
        check["sums_equal_single_rank"] = bool(check["sum_payoff_equal_single_rank"]
                                               and check["sum_payoff_sq_rel_diff"] < 1e-13
                                               and check["per_path_outputs_equal_single_rank"] is not False)
    # ---- throughput ----
    n_total = paths_per_gpu * world
    res = sharded.gbm_monte_carlo(key, n_total, cfg, math_mode=math_mode)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        res = sharded.gbm_monte_carlo(key, n_total, cfg, math_mode=math_mode)
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / iters
    exact = _black_scholes(cfg)
    value = float(n_total) * cfg["steps"] / (ms * 1e-3)
    int_peak = _native.measure_int32_alu_peak()
    return {"workload": "GBM Monte Carlo, Threefry in-kernel, path slabs by global path index", "n_gpus": world,
            "paths_total": n_total, "paths_per_gpu": paths_per_gpu, "steps": cfg["steps"], "math_mode": math_mode,
            "collective": "one NCCL all_reduce of 2 float64 per pass", "ms": ms, "path_steps_per_s": value,
            "price": res.price, "stderr": res.stderr, "black_scholes": exact,
            "sigmas_from_black_scholes": abs(res.price - exact) / res.stderr if res.stderr else None,
            "frac_of_int32_peak_per_gpu": value / world * GBM_INT_OPS_PER_PATH_STEP / int_peak, "check": check,
            "sums_equal_single_rank": check["sums_equal_single_rank"] if check else None}


def multi_gpu_gray_scott(rank: int, world: int, barrier, max_over_ranks, math_mode: str = "fast", cols: int = 16384,
                         halo: int = 16, steps_per_pass: int = 64, iters: int = 3) -> dict:
    """The stencil on `world` GPUs: row slabs on a periodic ring, boundary rows
    stored into the neighbours' ghost rows by the compute kernel (peer stores
    over NVLink, every copy engine load is an ordinary single-CTA one, nothing waits inside a kernel).  16384 x 16384 on 8
    GPUs (2048 rows per GPU); 8192 rows x 16384 columns per GPU otherwise.
    Checked in the same run: a 1024 x 16384 grid advanced 32 steps under SAFE by
    the slabs against rank 0 advancing the whole grid alone."""
    import torch

    from palladium_b200 import cuda_call_jit, families, sharded
    from palladium_b200 import workloads as W

    cfg = {k: v_ for k, v_ in W.GRAY_SCOTT_CONFIG.items() if k not in ("steps", "size", "seed")}
    # ---- the check ----
    rows_c, steps_c = 1024, 32
    rng = np.random.default_rng(11)
    u0 = (0.5 + 0.5 * rng.random((rows_c, cols), dtype=np.float32))
    v0 = (0.25 * rng.random((rows_c, cols), dtype=np.float32))
    lo, hi = sharded.partition(rows_c, world, rank)
    slab = sharded.GrayScottSlab(torch.from_numpy(u0[lo:hi]).cuda(), torch.from_numpy(v0[lo:hi]).cuda(), rows_c,
                                 halo=halo, constants=cfg, math_mode="safe", push=True)
    slab.advance(steps_c)
    su, sv = (t.clone() for t in slab.owned())
    pushes, exchanges = slab.pushes, slab.exchanges
    slab.close()
    equal = None
    if rows_c % world == 0:
        full_u, full_v = _gather_rows(su, world), _gather_rows(sv, world)
        if rank == 0:
            whole = cuda_call_jit(families.gray_scott(steps=steps_c, **cfg), grid=(rows_c, cols),
                                  out_shape=(_shaped((rows_c, cols)), _shaped((rows_c, cols))), math_mode="safe")
            wu, wv = whole(torch.from_numpy(u0).cuda(), torch.from_numpy(v0).cuda())
            equal = bool(torch.equal(full_u, wu) and torch.equal(full_v, wv))
    # ---- throughput ----
    rows_per_gpu = 2048 if world >= 8 else 8192
    rows_total = rows_per_gpu * world
    u = torch.rand((rows_per_gpu, cols), device="cuda") * 0.5 + 0.5
    v = torch.rand((rows_per_gpu, cols), device="cuda") * 0.25
    slab = sharded.GrayScottSlab(u, v, rows_total, halo=halo, constants=cfg, math_mode=math_mode, push=True)
    del u, v
    for _ in range(2):
        slab.advance(steps_per_pass)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        slab.advance(steps_per_pass)
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / iters
    finite = bool(torch.isfinite(slab.owned()[0]).all())
    slab.close()
    cell_steps = float(rows_total) * cols * steps_per_pass
    value = cell_steps / (ms * 1e-3)
    peak, note = _hbm_peak_gbs()
    gbs = value / world * GS_BYTES_PER_CELL_STEP / 1e9
    return {"workload": "Gray-Scott periodic 5-point stencil, row slabs", "n_gpus": world, "rows": rows_total,
            "cols": cols, "rows_per_gpu": rows_per_gpu, "halo": halo, "math_mode": math_mode,
            "exchange": f"boundary rows stored into the neighbours' ghost rows by the compute kernel every {halo} steps "
                        "(peer stores over NVLink), one 1-element all_reduce per exchange orders the calls",
            "steps_per_pass": steps_per_pass, "ms_per_pass": ms, "us_per_step": ms * 1e3 / steps_per_pass,
            "cell_steps_per_s": value, "algorithmic_gbs_per_gpu": gbs, "hbm_peak_gbs": peak,
            "frac_of_hbm_peak_per_gpu": gbs / peak, "peak_note": note, "finite": finite,
            "check": {"rows": rows_c, "cols": cols, "steps": steps_c, "math_mode": "safe", "pushes": pushes,
                      "point_to_point_exchanges": exchanges},
            "slab_equals_single_gpu": equal}


def multi_gpu_summary(rank: int, world: int, barrier, max_over_ranks, math_mode: str = "fast") -> dict:
    """The two families whose multi-GPU form has an exchange step, run by every
    rank of the job; the dict is meaningful on rank 0."""
    out = {}
    for name, fn in (("gbm", multi_gpu_gbm), ("gray_scott", multi_gpu_gray_scott)):
        try:
            out[name] = fn(rank, world, barrier, max_over_ranks, math_mode)
        except Exception as exc:   # every rank takes the same path: the failure is reported, the headline still prints
            out[name] = {"error": f"{type(exc).__name__}: {exc}"}
    return out


# ----------------------------------------------------------------------------- host <-> device copy ceiling
def host_copy_rates(rank: int, world: int, n_in: int = 100 << 20, n_out: int = 32 << 20, reps: int = 8) -> dict:
    """What the host-buffer path can at best achieve on this machine: plain
    cudaMemcpyAsync rates from / to pinned buffers of the sizes one RK4 pass moves
    (100 MB up, 32 MB down), per rank alone (the other ranks idle) and with every rank
    copying at once, each direction by itself and both together; then the
    host-buffer call itself with every rank calling at once.  Every rank takes part;
    the returned dict holds one list per figure, indexed by rank (on every rank)."""
    import torch
    import torch.distributed as dist

    from palladium_b200 import cuda_call_jit, families
    from palladium_b200 import workloads as W

    hin = torch.empty(n_in, dtype=torch.uint8).pin_memory()
    hin.fill_(1)
    hout = torch.empty(n_out, dtype=torch.uint8).pin_memory()
    hout.fill_(1)
    din = torch.empty(n_in, dtype=torch.uint8, device="cuda")
    dout = torch.empty(n_out, dtype=torch.uint8, device="cuda")
    up, down = torch.cuda.Stream(), torch.cuda.Stream()

    def h2d():
        din.copy_(hin, non_blocking=True)

    def d2h():
        hout.copy_(dout, non_blocking=True)

    def both():
        with torch.cuda.stream(up):
            din.copy_(hin, non_blocking=True)
        with torch.cuda.stream(down):
            hout.copy_(dout, non_blocking=True)

    def rate(fn, nbytes):   # GB/s over `reps` back-to-back copies
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        return nbytes * reps / (time.perf_counter() - t0) / 1e9

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    res = {}
    for r in range(world):          # one rank at a time
        sync()
        if r == rank:
            res["alone_h2d_gbs"], res["alone_d2h_gbs"] = rate(h2d, n_in), rate(d2h, n_out)
            res["alone_both_gbs"] = rate(both, n_in + n_out)
    sync()
    res["all_ranks_h2d_gbs"] = rate(h2d, n_in)
    sync()
    res["all_ranks_d2h_gbs"] = rate(d2h, n_out)
    sync()
    res["all_ranks_both_gbs"] = rate(both, n_in + n_out)
    sync()
    n = 1 << 22
    call = cuda_call_jit(families.lv_rk4(0.01, 1000), grid=(n,), out_shape=(_shaped((n,)), _shaped((n,))),
                         math_mode="fast")
    np_in = [torch.from_numpy(a).pin_memory().numpy() for a in W.lotka_volterra_ensemble(n, seed=17 + rank)]
    for _ in range(2):
        call(*np_in)
    sync()
    t0 = time.perf_counter()
    for _ in range(reps):
        call(*np_in)
    res["host_buffer_call_ms_all_ranks"] = (time.perf_counter() - t0) / reps * 1e3
    res["host_buffer_call_gbs"] = (sum(a.nbytes for a in np_in) + 8 * n) / (res["host_buffer_call_ms_all_ranks"] * 1e-3) / 1e9
    sync()
    if world > 1:
        everyone = [None] * world
        dist.all_gather_object(everyone, res)
    else:
        everyone = [res]
    return {k: [round(float(e[k]), 2) for e in everyone] for k in res}


# ----------------------------------------------------------------------------- as the main workload
def run(args, rank: int, local_rank: int, world: int, barrier, max_over_ranks) -> None:
    import torch

    from palladium_b200 import _native, sharded
    from palladium_b200 import workloads as W

    fma_peak = _native.measure_fp32_fma_peak()
    int_peak = _native.measure_int32_alu_peak()
    name = args.workload
    steps, warmup = args.steps, max(args.warmup, 3)
    line = {"n_gpus": world, "steps": steps, "warmup": warmup, "higher_is_better": True, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "cpu_baseline": None, "e2e": None, "gpu_launches": None}
    if name == "gbm":
        n_local = args.n or (1 << 24)
        n_total = n_local * world
        cfg = {k: v for k, v in W.GBM_CONFIG.items() if k not in ("n", "seed")}
        key = W.gbm_key(0)
        for _ in range(warmup):
            res = sharded.gbm_monte_carlo(key, n_total, cfg, math_mode=args.math_mode)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            res = sharded.gbm_monte_carlo(key, n_total, cfg, math_mode=args.math_mode)
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1)) / steps
        value = float(n_total) * cfg["steps"] / (ms * 1e-3)
        line.update({"metric": "gbm_path_steps_per_s", "value": value, "unit": "path-steps/s", "ms_per_step": ms,
                     "scaling": "weak", "dtype": "u32+f32", "gpu_launches": 2 * steps,
                     "config": {"workload": "gbm_threefry_monte_carlo", "paths_per_gpu": n_local, "steps": cfg["steps"],
                                "math_mode": args.math_mode, "collective": "one all_reduce of 2 float64 per step",
                                "price": res.price, "stderr": res.stderr,
                                "l2": "256 MB of per-path output per 2^26 paths; compute-bound"},
                     "roofline": {"bound": "int32_alu", "achieved": value / world * GBM_INT_OPS_PER_PATH_STEP / 1e12,
                                  "peak": int_peak / 1e12, "unit": "Tops/s",
                                  "frac": value / world * GBM_INT_OPS_PER_PATH_STEP / int_peak, "traffic": None,
                                  "peak_source": "add/xor/funnel-shift chain microbenchmark measured in this run"}})
    elif name == "gray_scott":
        size = args.n or 8192
        rows_total = size * world if world > 1 else size
        halo = int(getattr(args, "halo", 16))
        push = bool(getattr(args, "push", 1)) and world > 1
        lo, hi = sharded.partition(rows_total, world, rank)
        u = torch.rand((hi - lo, size), device="cuda") * 0.5 + 0.5
        v = torch.rand((hi - lo, size), device="cuda") * 0.25
        cfg = {k: v_ for k, v_ in W.GRAY_SCOTT_CONFIG.items() if k not in ("steps", "size", "seed")}
        slab = sharded.GrayScottSlab(u, v, rows_total, halo=halo, constants=cfg, math_mode=args.math_mode, push=push)
        per_step = 64
        for _ in range(warmup):
            slab.advance(per_step)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            slab.advance(per_step)
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1)) / steps
        cell_steps = float(rows_total) * size * per_step
        value = cell_steps / (ms * 1e-3)
        peak, note = _hbm_peak_gbs()
        gbs = value / world * GS_BYTES_PER_CELL_STEP / 1e9
        line.update({"metric": "gray_scott_cell_steps_per_s", "value": value, "unit": "cell-steps/s", "ms_per_step": ms,
                     "scaling": "weak", "gpu_launches": steps * per_step,
                     "config": {"workload": "gray_scott_periodic", "rows": rows_total, "cols": size,
                                "stencil_steps_per_bench_step": per_step, "halo": halo, "math_mode": args.math_mode,
                                "parallelism": f"row slabs x{world}, halo exchange every {halo} steps"
                                               + (" from inside the compute kernel (peer stores over NVLink)" if push
                                                  else " (point-to-point sends)" if world > 1 else ""),
                                "l2": "fields are 268 MB each at 8192^2, larger than the 126 MB L2"},
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                  "traffic": None, "peak_source": note}})
    elif name == "vdp_bs32":
        n = args.n or (1 << 20)
        r = bench_vdp(n, args.math_mode, warmup=warmup, iters=steps, fma_peak=fma_peak)
        ms = max_over_ranks(r["ms"])
        value = r["attempts"] * world / (ms * 1e-3)
        line.update({"metric": "bs32_attempted_steps_per_s", "value": value, "unit": "attempted steps/s",
                     "ms_per_step": ms, "scaling": "weak", "gpu_launches": steps, "config": {"workload": "vdp_bs32", **r},
                     "roofline": {"bound": "fp32_fma", "achieved": r["attempts_per_s"] * VDP_FLOPS_PER_ATTEMPT / 1e12,
                                  "peak": fma_peak / 1e12, "unit": "TFLOP/s", "frac": r.get("frac_of_fp32_peak"),
                                  "traffic": None}})
    elif name == "kepler_df32":
        n = args.n or (1 << 20)
        r = bench_kepler(n, 1000, warmup=1, iters=steps, fma_peak=fma_peak)
        ms = max_over_ranks(r["ms"])
        value = float(n) * world * 1000 / (ms * 1e-3)
        line.update({"metric": "df32_trajectory_steps_per_s", "value": value, "unit": "trajectory-steps/s",
                     "ms_per_step": ms, "scaling": "weak", "gpu_launches": steps, "config": {"workload": "kepler_df32", **r},
                     "roofline": {"bound": "fp32_fma", "achieved": r["trajectory_steps_per_s"] * DF32_KEPLER_FLOPS / 1e12,
                                  "peak": fma_peak / 1e12, "unit": "TFLOP/s", "frac": r.get("frac_of_fp32_peak"),
                                  "traffic": None}})
    elif name == "custom_ode":
        n = args.n or (1 << 22)
        r = bench_custom_ode(n, 1000, args.math_mode, warmup=warmup, iters=steps, fma_peak=fma_peak)
        ms = max_over_ranks(r["ms"])
        value = float(n) * world * 1000 / (ms * 1e-3)
        line.update({"metric": "rk4_ensemble_trajectory_steps_per_s", "value": value, "unit": "trajectory-steps/s",
                     "ms_per_step": ms, "scaling": "weak", "gpu_launches": steps,
                     "config": {"workload": "custom_ode_lotka_volterra", **r},
                     "roofline": {"bound": "fp32_fma", "achieved": r["trajectory_steps_per_s"] * 58 / 1e12,
                                  "peak": fma_peak / 1e12, "unit": "TFLOP/s", "frac": r.get("frac_of_fp32_peak"),
                                  "traffic": None}})
    elif name == "host_copies":
        rates = host_copy_rates(rank, world)
        total = sum(rates["host_buffer_call_gbs"])
        line.update({"metric": "host_buffer_call_bytes_per_s", "value": total * 1e9, "unit": "B/s", "scaling": "weak",
                     "ms_per_step": max(rates["host_buffer_call_ms_all_ranks"]), "dtype": "u8", "gpu_launches": None,
                     "config": {"workload": "host <-> device copy rates behind the host-buffer call, per rank",
                                "bytes_up_per_pass": 100 << 20, "bytes_down_per_pass": 32 << 20, **rates}})
    elif name == "full":
        line.update(full_configs(fma_peak, int_peak))
    else:
        raise SystemExit(f"unknown workload {name!r}")
    if rank == 0:
        print(json.dumps(line), flush=True)
