"""Per-thread adaptive stepping (the reference's examples/02_adaptive_lockstep.py).

A mild Van der Pol ensemble salted with a few stiff members, integrated by the
Bogacki-Shampine 3(2) + PI-controller kernel: each trajectory takes its own
steps, and lanes that finish early are refilled with new trajectories.
"""

import time

import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))  # run from a source checkout

import palladium_b200 as pd  # noqa: E402
from palladium_b200 import families, pl  # noqa: E402

N = 2048
STIFF_FRACTION = 0.02
CFG = dict(t1=10.0, rtol=1e-5, atol=1e-7, dt0=0.01, max_steps=6000)


def solver(n, **controller):
    spec_1 = pl.BlockSpec((1,), lambda i: (i,))
    return pd.cuda_call(
        families.vdp_bs32(**CFG, **controller),
        grid=(n,),
        in_specs=[spec_1] * 3,
        out_specs=(spec_1,) * 6,
        out_shape=tuple(pl.ShapeDtypeStruct((n,), np.float32) for _ in range(6)),
        math_mode=pd.MathMode.RELAXED,
    )


def main():
    rng = np.random.default_rng(3)
    mild = rng.uniform(0.5, 2.0, N).astype(np.float32)
    mixed = mild.copy()
    k = int(N * STIFF_FRACTION)
    mixed[rng.choice(N, k, replace=False)] = rng.uniform(300.0, 500.0, k)
    x0, v0 = np.full(N, 2.0, np.float32), np.zeros(N, np.float32)
    solve = solver(N)
    solve(x0, v0, mild)
    for label, mu in (("all mild", mild), (f"{k} stiff members", mixed)):
        t0 = time.perf_counter()
        t, x, v, steps, rejected, real = solve(x0, v0, mu)
        dt = time.perf_counter() - t0
        print(f"{label:18s} {dt * 1e3:7.2f} ms  accepted steps median {int(np.median(real))}, max {int(real.max())}; "
              f"rejected mean {rejected.mean():.1f}; all reached t1: {bool(np.all(np.abs(t - CFG['t1']) < 1e-4))}")
    _, _, _, _, rejected_i, _ = solver(N, pcoeff=0.0, icoeff=1.0)(x0, v0, mixed)
    _, _, _, _, rejected_pi, _ = solve(x0, v0, mixed)
    print(f"controller check on the mixed ensemble: I-only rejects {rejected_i.mean():.1f} per trajectory, "
          f"PI rejects {rejected_pi.mean():.1f}")


if __name__ == "__main__":
    main()
