"""Massive ensembles of small ODEs (the reference's examples/01_ode_ensembles.py).

One GPU thread integrates one Lotka-Volterra system (RK4, fixed step) with its
own parameters; the grid is the ensemble.  The call is the reference's
`metal_call(lv_kernel, grid=(n,), in_specs=[spec_1]*6, ...)` with the kernel
family in place of the Pallas function.
"""

import time

import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))  # run from a source checkout

import palladium_b200 as pd  # noqa: E402
from palladium_b200 import families, pl  # noqa: E402

DT, STEPS = 0.01, 500
N = 100_000


def ensemble(n, seed=17):
    rng = np.random.default_rng(seed)
    ranges = ((0.8, 1.2), (0.8, 1.2), (0.9, 1.3), (0.3, 0.5), (0.08, 0.12), (0.3, 0.5))  # x0, y0, a, b, c, d
    return tuple(rng.uniform(lo, hi, n).astype(np.float32) for lo, hi in ranges)


def solver(n, math_mode=pd.MathMode.FAST):
    spec_1 = pl.BlockSpec((1,), lambda i: (i,))
    return pd.cuda_call(
        families.lv_rk4(DT, STEPS),
        grid=(n,),
        in_specs=[spec_1] * 6,
        out_specs=(spec_1, spec_1),
        out_shape=(pl.ShapeDtypeStruct((n,), np.float32), pl.ShapeDtypeStruct((n,), np.float32)),
        math_mode=math_mode,
    )


def main():
    args = ensemble(N)
    solve = solver(N)
    print(solve.explain(*args))
    solve(*args), solve(*args)  # binding and pinned-buffer warm-up outside the clock
    t0 = time.perf_counter()
    x, y = solve(*args)
    dt = time.perf_counter() - t0
    print(f"Lotka-Volterra ensemble: N={N}, RK4, {STEPS} steps of dt={DT}: {dt * 1e3:.2f} ms end to end "
          f"({N * STEPS / dt / 1e9:.1f} G trajectory-steps/s), x[0]={x[0]:.6f}, y[0]={y[0]:.6f}")
    pinned = solve.pin(*args)  # inputs stay on the device
    t0 = time.perf_counter()
    pinned()
    print(f"pinned inputs: {(time.perf_counter() - t0) * 1e3:.2f} ms")


if __name__ == "__main__":
    main()
