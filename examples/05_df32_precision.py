"""Does compensated arithmetic buy real accuracy (the reference's
examples/05_df32_precision.py): the RK4 Lotka-Volterra ensemble as FAST float32,
SAFE float32 and df32, each measured against a float64 NumPy integration."""

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
    ranges = ((0.8, 1.2), (0.8, 1.2), (0.9, 1.3), (0.3, 0.5), (0.08, 0.12), (0.3, 0.5))
    return tuple(rng.uniform(lo, hi, n).astype(np.float32) for lo, hi in ranges)


def float64_reference(x0, y0, a, b, c, d, dt):
    x, y = x0.astype(np.float64), y0.astype(np.float64)
    a, b, c, d = (v.astype(np.float64) for v in (a, b, c, d))
    rhs = lambda x, y: (a * x - b * x * y, c * x * y - d * y)  # noqa: E731
    for _ in range(STEPS):
        k1x, k1y = rhs(x, y)
        k2x, k2y = rhs(x + 0.5 * dt * k1x, y + 0.5 * dt * k1y)
        k3x, k3y = rhs(x + 0.5 * dt * k2x, y + 0.5 * dt * k2y)
        k4x, k4y = rhs(x + dt * k3x, y + dt * k3y)
        x = x + dt / 6.0 * (k1x + 2 * k2x + 2 * k3x + k4x)
        y = y + dt / 6.0 * (k1y + 2 * k2y + 2 * k3y + k4y)
    return x, y


def run(family, math_mode, args):
    spec_1 = pl.BlockSpec((1,), lambda i: (i,))
    shape = pl.ShapeDtypeStruct((N,), np.float32)
    call = pd.cuda_call(family, grid=(N,), in_specs=[spec_1] * 6, out_specs=(spec_1, spec_1),
                        out_shape=(shape, shape), math_mode=math_mode)
    return call(*args)


def main():
    args = ensemble(N)
    # the df32 kernel receives dt as a float32 scalar, so the float64 truth uses that value
    want_x, want_y = float64_reference(*args, dt=float(np.float32(DT)))
    errs = {}
    for label, family, mode in (("float32, FAST", families.lv_rk4(DT, STEPS), pd.MathMode.FAST),
                                ("float32, SAFE", families.lv_rk4(DT, STEPS), pd.MathMode.SAFE),
                                ("df32, SAFE", families.lv_rk4_df32(DT, STEPS), pd.MathMode.SAFE)):
        x, y = run(family, mode, args)
        errs[label] = max(np.max(np.abs(x - want_x)), np.max(np.abs(y - want_y)))
        print(f"  {label:<14} max abs error vs float64: {errs[label]:.2e}")
    assert errs["df32, SAFE"] < errs["float32, FAST"], "df32 should be more accurate than plain FAST float32"


if __name__ == "__main__":
    main()
