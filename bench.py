"""Benchmark of the ensemble-integrator hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload rk4_lv|vdp_bs32|gbm|gray_scott|kepler_df32|custom_ode|host_copies] [--n N_PER_GPU]

One "step" is one pass of a kernel family over one batch of synthetic input.
The default workload is the headline one: the fixed-step RK4 Lotka-Volterra
ensemble (dt = 0.01, 1000 RK4 steps per trajectory), sized for throughput at
2^22 trajectories per GPU (weak scaling: each rank integrates its own slab of
trajectories, no collective on the data path).  Rank 0 prints ONE JSON line.

Timed regions
  value : K steps with inputs resident in HBM, CUDA events on the launch stream,
          barrier + synchronise on both sides, max over ranks.
  e2e   : the same K steps through the host-buffer C-ABI call (pd_dispatch_host,
          what an XLA:CPU FFI handler would be given): every step uploads its
          inputs from pinned host memory, runs, and downloads its outputs.
  cpu_baseline / --impl reference : the reference's own emitted RK4 kernel
          (tests/golden/rk4_lotka_volterra.metal compiled for the CPU by
          oracle/build.py) on all host cores, or the oracle port where the
          reference has no compiled form; a bounded sample of the workload.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LV_STEPS = 1000
LV_DT = 0.01
LV_FLOPS_PER_TRAJ_STEP = 58  # float operations in the reference kernel's loop body
                             # (tests/golden/rk4_lotka_volterra.metal:58-258 in the reference)
SM_COUNT = 148
# What each math mode of the RK4 kernel is held to against the CPU oracle, and the GPU test that asserts it.
PARITY = {
    "safe": {"against_oracle": "bit-exact final states", "test": "tests/test_gpu_parity.py::test_rk4_named_configuration_safe_is_bit_exact"},
    "relaxed": {"against_oracle": ">= 95 % of final states within rtol 1e-5, every state within 1e-4 (fused multiply-adds "
                                  "round differently per operation); error against float64 no larger than the oracle's",
                "test": "tests/test_gpu_parity.py::test_rk4_named_configuration_fast_modes"},
    "fast": {"against_oracle": ">= 95 % of final states within rtol 1e-5, every state within 1e-4 (the kernel integrates the "
                               "rescaled state X = c x, Y = b y); error against float64 no larger than the oracle's; "
                               "the mode that meets rtol 1e-5 on every state is safe, timed in families.rk4_lv_safe",
             "test": "tests/test_gpu_parity.py::test_rk4_named_configuration_fast_modes"},
}
FP32_LANES_PER_SM = 128


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="rk4_lv")
    ap.add_argument("--n", type=int, default=0, help="units per GPU (0 = workload default)")
    ap.add_argument("--push", type=int, default=1,
                    help="gray_scott on several GPUs: 1 = halo rows stored into the neighbours' memory by the "
                         "compute kernel, 0 = point-to-point exchange between calls")
    ap.add_argument("--halo", type=int, default=16, help="gray_scott on several GPUs: ghost rows per side")
    ap.add_argument("--math-mode", default="fast", choices=["safe", "relaxed", "fast"])
    ap.add_argument("--no-families", action="store_true", help="skip the short per-family measurements")
    ap.add_argument("--no-named", action="store_true",
                    help="skip the full-size named configurations of the other families (about 20 s)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="set a native tuning knob (pd_set_tuning), e.g. --tune vdp_variant=0")
    return ap.parse_args()


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs."""

    REASONS = {
        0x8: "hw_slowdown",
        0x40: "hw_thermal_slowdown",
        0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_rk4(n_sample: int, threads: int | None = None):
    """Time the reference's emitted RK4 kernel (or the oracle port) on the host.
    Returns (traj_steps_per_s, kind, cores, sample description)."""
    import oracle
    from palladium_b200 import workloads as W

    cores = len(os.sched_getaffinity(0))
    if threads:
        cores = threads
    oracle.set_threads(cores)
    args = W.lotka_volterra_ensemble(n_sample, seed=17)
    if oracle.reference_lib() is not None:
        # The golden kernel is 500 steps of dt = 0.01; two chained calls are the 1000-step workload.
        kind = "reference"
        oracle.lv_rk4_reference_golden(*[a[:4096] for a in args])  # warm the thread pool
        t0 = time.perf_counter()
        x, y = oracle.lv_rk4_reference_golden(*args)
        oracle.lv_rk4_reference_golden(x, y, *args[2:])
        dt = time.perf_counter() - t0
    else:
        kind = "port"
        oracle.lv_rk4(*[a[:4096] for a in args], dt=LV_DT, steps=10)
        t0 = time.perf_counter()
        oracle.lv_rk4(*args, dt=LV_DT, steps=LV_STEPS)
        dt = time.perf_counter() - t0
    rate = n_sample * LV_STEPS / dt
    return rate, kind, cores, f"{n_sample} trajectories x {LV_STEPS} steps of the same ensemble, one pass, {dt:.2f} s"


def cpu_family_baselines() -> dict:
    """The CPU oracle (the port of each reference kernel) timed on all host cores
    on a bounded sample of each family's workload: the reported CPU baseline of
    the families other than the headline one."""
    import oracle
    from palladium_b200 import workloads as W

    cores = len(os.sched_getaffinity(0))
    oracle.set_threads(cores)
    out = {"cores": cores, "kind": "port"}

    def timed(fn):
        t0 = time.perf_counter()
        res = fn()
        return time.perf_counter() - t0, res

    n = 4096
    x0, v0, mu = W.van_der_pol_ensemble(n)
    cfg = {k: v for k, v in W.VDP_CONFIG.items() if k not in ("n", "seed")}
    sec, res = timed(lambda: oracle.vdp_bs32(x0, v0, mu, pow="libm", **cfg))
    attempts = float((res[4] + res[5]).sum())
    out["vdp_bs32"] = {"sample": f"{n} trajectories, full {cfg['max_steps']}-iteration loop as the reference runs it",
                       "seconds": sec, "attempts_per_s": attempts / sec,
                       "loop_iterations_per_s": n * cfg["max_steps"] / sec}
    n = 1 << 17
    gcfg = {k: v for k, v in W.GBM_CONFIG.items() if k not in ("n", "seed")}
    sec, _ = timed(lambda: oracle.gbm(W.gbm_key(0), n, **gcfg))
    out["gbm"] = {"sample": f"{n} paths x {gcfg['steps']} steps", "seconds": sec,
                  "path_steps_per_s": n * gcfg["steps"] / sec}
    size, steps = 2048, 20
    u = (np.random.default_rng(0).random((size, size)) * 0.5 + 0.5).astype(np.float32)
    v = (np.random.default_rng(1).random((size, size)) * 0.25).astype(np.float32)
    sec, _ = timed(lambda: oracle.gray_scott(u, v, steps=steps))
    out["gray_scott"] = {"sample": f"{size} x {size}, {steps} steps", "seconds": sec,
                         "cell_steps_per_s": size * size * steps / sec}
    # the job of the reference's CPU comparison (benchmarks/bench_ensembles.py:88-118: Tsit5 under a step
    # controller, rtol 1e-6, atol 1e-8, t = 5, n = 10 000 and 100 000), on the CPU restatement of the same pair
    from oracle import custom_ode as oracle_custom
    import bench_families as bf

    for n in (10_000, 100_000):
        ens = bf.reference_benchmark_ensemble(n)
        kw = dict(method="tsit5", t1=5.0, rtol=1e-6, atol=1e-8, dt0=0.01, max_steps=bf.LV_TSIT5_MAX_STEPS)
        oracle_custom.erk(bf.LV_RHS, 2, 4, [a[:256] for a in ens], **kw)       # builds the shared object
        sec, res = timed(lambda: oracle_custom.erk(bf.LV_RHS, 2, 4, ens, **kw))
        out[f"lv_tsit5_n={n}"] = {"sample": f"{n} trajectories to t = 5 (the whole job), loop of {kw['max_steps']} iterations "
                                            "(no trajectory needs more than 48)",
                                  "seconds": sec, "ms": sec * 1e3, "accepted_steps_mean": float(res[5].mean())}
    n, steps = 8192, 500
    _, pairs = W.kepler_ensemble(n)
    sec, _ = timed(lambda: oracle.kepler_rk4_df32(pairs, dt=1e-3, steps=steps))
    out["kepler_df32"] = {"sample": f"{n} orbits x {steps} steps", "seconds": sec,
                          "trajectory_steps_per_s": n * steps / sec}
    return out



def run_reference_arm(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    n_sample = 1 << 19
    rates = []
    sample = ""
    for _ in range(args.warmup):
        cpu_rk4(1 << 16)
    t_all = time.perf_counter()
    for _ in range(args.steps):
        rate, kind, cores, sample = cpu_rk4(n_sample)
        rates.append(rate)
        if time.perf_counter() - t_all > 150:
            break
    value = float(np.mean(rates))
    line = {
        "impl": "reference", "metric": "rk4_ensemble_trajectory_steps_per_s", "value": value,
        "unit": "trajectory-steps/s", "n_gpus": args.gpus, "steps": len(rates), "warmup": args.warmup,
        "ms_per_step": 1e3 * n_sample * LV_STEPS / value, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "rk4_lotka_volterra", "dt": LV_DT, "rk4_steps": LV_STEPS,
                   "trajectories_per_step": n_sample, "runs_on": "host cores"},
        "cpu_baseline": {"value": value, "unit": "trajectory-steps/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "trajectory-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    rank, local_rank, world = dist_env()

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import palladium_b200 as pd
    from palladium_b200 import _native, families, pl, workloads as W

    for item in args.tune:
        key, _, val = item.partition("=")
        _native.set_tuning(key, int(val))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.workload != "rk4_lv":
        import bench_families

        bench_families.run(args, rank, local_rank, world, barrier, max_over_ranks)
        if world > 1:
            dist.destroy_process_group()
        return

    n = args.n or (1 << 22)
    mode = pd.MathMode(args.math_mode)
    spec1 = pl.BlockSpec((1,), lambda i: (i,))
    shaped = pl.ShapeDtypeStruct((n,), np.float32)
    call = pd.cuda_call_jit(families.lv_rk4(LV_DT, LV_STEPS), grid=(n,), in_specs=[spec1] * 6,
                            out_specs=(spec1, spec1), out_shape=(shaped, shaped), math_mode=mode)
    # Each rank integrates its own slab of one global ensemble: same generator,
    # seed offset by rank (trajectories are independent, so slabs need no exchange).
    host_in = W.lotka_volterra_ensemble(n, seed=17 + rank)
    dev_in = [torch.from_numpy(a).cuda() for a in host_in]

    # ---- device-resident throughput -------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        out = call(*dev_in)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for _ in range(args.steps):
            out = call(*dev_in)
        e1.record()
        barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = ms_total / args.steps
    total_traj_steps = float(n) * LV_STEPS * world
    value = total_traj_steps / (ms_per_step * 1e-3)

    # ---- roofline of the dominant (only) kernel --------------------------------------
    kernel_ms = ms_per_step  # one kernel per step; the events bracket only those launches
    fma_peak = _native.measure_fp32_fma_peak()
    achieved_flops = float(n) * LV_STEPS * LV_FLOPS_PER_TRAJ_STEP / (kernel_ms * 1e-3)
    clk = clocks.summary()
    nominal_peak = 2.0 * FP32_LANES_PER_SM * SM_COUNT * (clk["sm_max_mhz"] or 1965) * 1e6
    roofline = {
        "bound": "fp32_fma", "achieved": achieved_flops / 1e12, "peak": fma_peak / 1e12, "unit": "TFLOP/s",
        "frac": achieved_flops / fma_peak,
        # ncu on an N = 1 212 416 capture: dram__bytes_read = 24 B x N exactly (each input array read
        # once), writes 8 B x N once evicted from L2; scaled by N for this launch.
        "traffic": 32 * n,
        "peak_source": "FMA-chain microbenchmark of this library, measured in this run on this GPU "
                       "(MEASURED_PEAKS.json holds no fp32 figure)",
        "nominal_peak": nominal_peak / 1e12, "frac_of_nominal": achieved_flops / nominal_peak,
        "flops_per_trajectory_step": LV_FLOPS_PER_TRAJ_STEP, "kernel_ms": kernel_ms,
        "hbm_bytes_per_launch_algorithmic": 32 * n,
    }

    # ---- end to end through the host-buffer C-ABI call --------------------------------
    pinned_in = [torch.from_numpy(a).pin_memory() for a in host_in]
    np_in = [t.numpy() for t in pinned_in]
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        res = call(*np_in)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        res = call(*np_in)
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    checksum = float(res[0][:8].sum())
    e2e = {"value": total_traj_steps / (e2e_ms * 1e-3), "unit": "trajectory-steps/s",
           "h2d_bytes_per_step": int(sum(a.nbytes for a in np_in)), "d2h_bytes_per_step": int(8 * n),
           "ms_per_step": e2e_ms, "steps": e2e_steps, "checksum": checksum,
           "path": "cuda_call_jit(host arrays) -> pd_dispatch_host: pinned host inputs and outputs; the call cuts the "
                   "ensemble into ~32 chunks over 6 streams so upload, kernel and download overlap"}

    # ---- named configuration (N = 100 000), device-resident ---------------------------
    named = None
    cpu_baseline = None
    fam = None
    if rank == 0:
        n_named = 100_000
        shaped_n = pl.ShapeDtypeStruct((n_named,), np.float32)
        call_n = pd.cuda_call_jit(families.lv_rk4(LV_DT, LV_STEPS), grid=(n_named,), out_shape=(shaped_n, shaped_n),
                                  math_mode=mode)
        dn = [torch.from_numpy(a).cuda() for a in W.lotka_volterra_ensemble(n_named, seed=17)]
        for _ in range(5):
            call_n(*dn)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(50):
            call_n(*dn)
        a1.record()
        torch.cuda.synchronize()
        ms_named = a0.elapsed_time(a1) / 50
        named = {"trajectories": n_named, "rk4_steps": LV_STEPS, "ms_per_pass": ms_named,
                 "value": n_named * LV_STEPS / (ms_named * 1e-3),
                 "frac_of_fma_peak": n_named * LV_STEPS * LV_FLOPS_PER_TRAJ_STEP / (ms_named * 1e-3) / fma_peak}
        if not args.no_cpu:
            rate, kind, cores, sample = cpu_rk4(1 << 20)
            cpu_baseline = {"value": rate, "unit": "trajectory-steps/s", "cores": cores, "kind": kind, "sample": sample}
            one, _, _, one_sample = cpu_rk4(1 << 16, threads=1)   # the same code on a single host thread
            cpu_baseline["single_thread"] = {"value": one, "cores": 1, "sample": one_sample}
        if world == 1 and not args.no_families:
            try:
                import bench_families

                fam = bench_families.quick_summary(named=not args.no_named)
                if not args.no_cpu:
                    fam["cpu_baselines"] = cpu_family_baselines()
            except Exception as exc:  # the headline line must still be printed
                fam = {"error": f"{type(exc).__name__}: {exc}"}
    if world > 1 and not args.no_families:
        # The two families whose multi-GPU form has an exchange step (the Monte Carlo's all-reduce, the
        # stencil's halo rows), each with a check against a single-rank result; every rank takes part.
        import bench_families

        fam = bench_families.multi_gpu_summary(rank, world, barrier, max_over_ranks, args.math_mode)

    if rank == 0:
        line = {
            "metric": "rk4_ensemble_trajectory_steps_per_s", "value": value, "unit": "trajectory-steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "rk4_lotka_volterra", "dt": LV_DT, "rk4_steps": LV_STEPS,
                       "trajectories_per_gpu": n, "math_mode": args.math_mode, "parallelism": f"trajectory slabs x{world}",
                       "parity": PARITY[args.math_mode],
                       "l2": "inputs + outputs are 32 B x N = 134 MB per pass, larger than the 126 MB L2; the kernel is compute-bound"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": args.steps,
            "clocks": clk, "named_config": named, "families": fam,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
