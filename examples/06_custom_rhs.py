"""A right-hand side of your own (no counterpart among the reference's examples;
it stands where the reference lets a user write any Pallas function).

The Lorenz system, one thread per parameter set: the right-hand side is three
lines of CUDA C, compiled at run time under the call's math mode and cached.
Run once with fixed-step RK4, once with the adaptive Bogacki-Shampine 3(2)
controller the Van der Pol example uses, and once with Tsitouras' 5(4) pair (the
method the reference's CPU comparison integrates with) under the same controller.
"""

import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))  # run from a source checkout

import palladium_b200 as pd  # noqa: E402
from palladium_b200 import families, pl  # noqa: E402

LORENZ = """
dy[0] = p[0] * (y[1] - y[0]);
dy[1] = y[0] * (p[1] - y[2]) - y[1];
dy[2] = y[0] * y[1] - p[2] * y[2];
"""
N = 200_000


def ensemble(n, seed=23):
    rng = np.random.default_rng(seed)
    state = [rng.uniform(-5, 5, n).astype(np.float32) for _ in range(3)]
    params = [rng.uniform(9, 11, n).astype(np.float32),      # sigma
              rng.uniform(20, 30, n).astype(np.float32),     # rho
              rng.uniform(2.0, 3.0, n).astype(np.float32)]   # beta
    return state + params


def solver(n, n_out, **constants):
    spec_1 = pl.BlockSpec((1,), lambda i: (i,))
    return pd.cuda_call(
        families.custom_ode(LORENZ, dim=3, nparam=3, **constants),
        grid=(n,),
        in_specs=[spec_1] * 6,
        out_specs=(spec_1,) * n_out,
        out_shape=tuple(pl.ShapeDtypeStruct((n,), np.float32) for _ in range(n_out)),
        math_mode=pd.MathMode.RELAXED,
    )


def timed(call, args, repeats=3):
    """Result and the best end-to-end time of a few calls (the first ones still set up pinned buffers)."""
    best, out = float("inf"), None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = call(*args)
        best = min(best, time.perf_counter() - t0)
    return out, best * 1e3


def main():
    args = ensemble(N)
    fixed = solver(N, 3, method="rk4", dt=0.002, steps=1000)
    print(fixed.explain(*args))
    fixed(*args)  # compile + warm-up
    (x, y, z), ms = timed(fixed, args)
    print(f"Lorenz RK4: N={N}, 1000 steps: {ms:.2f} ms end to end, "
          f"state[0]=({x[0]:.4f}, {y[0]:.4f}, {z[0]:.4f})")
    adaptive = solver(N, 7, method="bs32", t1=2.0, rtol=1e-5, atol=1e-7, dt0=1e-3, max_steps=20_000)
    adaptive(*args)
    (t, x2, y2, z2, steps, rejected, real), ms = timed(adaptive, args)
    print(f"Lorenz BS3(2): {ms:.2f} ms end to end, all reached t1: {bool(np.all(t == 2.0))}, "
          f"accepted steps {real.min():.0f}..{real.max():.0f}, rejected up to {rejected.max():.0f}, "
          f"|RK4 - adaptive| median {np.median(np.abs(x - x2)):.2e}")
    tsit5 = solver(N, 7, method="tsit5", t1=2.0, rtol=1e-5, atol=1e-7, dt0=1e-3, max_steps=20_000)
    tsit5(*args)
    (t, x3, _, _, _, rejected5, real5), ms = timed(tsit5, args)
    print(f"Lorenz Tsit5:  {ms:.2f} ms end to end, all reached t1: {bool(np.all(t == 2.0))}, "
          f"accepted steps {real5.min():.0f}..{real5.max():.0f} (BS3(2) needed {real.min():.0f}..{real.max():.0f}), "
          f"|BS3(2) - Tsit5| median {np.median(np.abs(x2 - x3)):.2e}")


if __name__ == "__main__":
    main()
