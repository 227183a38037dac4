"""SDE Monte Carlo (the reference's examples/03_sde_montecarlo.py): a European
call under geometric Brownian motion, one thread per path, RNG in the kernel,
checked against Black-Scholes.  Two kernels, as in the reference: the cheap
pcg_hash counter RNG and Threefry-2x32-20 keyed per (path, step)."""

import time
from math import erf, exp, log, sqrt

import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))  # run from a source checkout

import palladium_b200 as pd  # noqa: E402
from palladium_b200 import families, pl  # noqa: E402

N_PATHS = 1 << 20
N_STEPS = 256
S0, K, T, R, SIGMA = 100.0, 105.0, 1.0, 0.03, 0.2


def black_scholes_call(s0, k, t, r, sigma):
    cdf = lambda x: 0.5 * (1.0 + erf(x / sqrt(2.0)))  # noqa: E731
    d1 = (log(s0 / k) + (r + sigma**2 / 2) * t) / (sigma * sqrt(t))
    return s0 * cdf(d1) - k * exp(-r * t) * cdf(d1 - sigma * sqrt(t))


def report(label, payoff, seconds):
    price = float(np.exp(-R * T) * payoff.mean())
    stderr = float(np.exp(-R * T) * payoff.std(ddof=1) / np.sqrt(payoff.size))
    exact = black_scholes_call(S0, K, T, R, SIGMA)
    print(f"  {label}: {price:.4f} +/- {stderr:.4f} in {seconds * 1e3:.2f} ms "
          f"({N_PATHS * N_STEPS / seconds / 1e9:.1f} Gsteps/s), {abs(price - exact) / stderr:.1f} sigma from "
          f"Black-Scholes ({exact:.4f})")
    assert abs(price - exact) < 5 * stderr, f"{label}: MC price off by >5 sigma"


def main():
    constants = dict(s0=S0, strike=K, r=R, sigma=SIGMA, t=T, steps=N_STEPS)
    out = pl.ShapeDtypeStruct((N_PATHS,), np.float32)
    hand = pd.cuda_call(families.gbm_pcg(**constants), grid=(N_PATHS,), out_shape=out)
    hand(), hand()  # binding, context and pinned-buffer warm-up outside the clock
    t0 = time.perf_counter()
    payoff = hand()
    t_hand = time.perf_counter() - t0
    report("pcg_hash", payoff, t_hand)

    threefry = pd.cuda_call(families.gbm_threefry(**constants), grid=(N_PATHS,),
                            in_specs=[pl.BlockSpec((2,), lambda i: (0,))],
                            out_specs=pl.BlockSpec((1,), lambda i: (i,)), out_shape=out)
    seed = np.array([0, 0], np.uint32)  # key data of an integer seed 0: (high word, low word)
    threefry(seed), threefry(seed)
    t0 = time.perf_counter()
    payoff = threefry(seed)
    t_fry = time.perf_counter() - t0
    report("Threefry", payoff, t_fry)
    print(f"  Threefry / pcg_hash slowdown: {t_fry / t_hand:.1f}x")


if __name__ == "__main__":
    main()
