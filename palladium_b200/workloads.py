"""Seeded synthetic inputs for the five benchmark configurations.

The reference draws its ensembles with `np.random.default_rng(seed)` and casts
each draw to float32 (examples/01_ode_ensembles.py:20-29); the generators here
follow that pattern with the distributions of the benchmark configurations.
Every array is float32 (uint32 for RNG keys), C-contiguous, structure-of-arrays.
"""

from __future__ import annotations

import numpy as np

__all__ = [
    "lotka_volterra_ensemble",
    "van_der_pol_ensemble",
    "gbm_key",
    "GBM_CONFIG",
    "gray_scott_initial_state",
    "GRAY_SCOTT_CONFIG",
    "kepler_ensemble",
    "split_df32",
    "join_df32",
    "kepler_energy",
    "LV_CONFIG",
    "VDP_CONFIG",
    "KEPLER_CONFIG",
]

LV_CONFIG = dict(dt=0.01, steps=1000, n=100_000, seed=17)
VDP_CONFIG = dict(t1=20.0, rtol=1e-6, atol=1e-8, dt0=1e-3, max_steps=100_000, pcoeff=0.4, icoeff=0.3,
                  safety=0.9, factor_min=0.2, factor_max=10.0, error_order=3, n=1_000_000, seed=3)
GBM_CONFIG = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=252, n=1 << 26, seed=0)
GRAY_SCOTT_CONFIG = dict(du=0.16, dv=0.08, f=0.035, k=0.065, dt=1.0, steps=10_000, size=8192, seed=11)
KEPLER_CONFIG = dict(dt=1e-3, gm=1.0, steps=100_000, n=1_000_000, seed=5)


def lotka_volterra_ensemble(n: int, seed: int = 17):
    """(x0, y0, a, b, c, d) for dx = a x - b x y, dy = c x y - d y.

    x0, y0 ~ U[0.5, 2); alpha ~ U[0.8, 1.2), beta ~ U[0.3, 0.5),
    gamma ~ U[2.5, 3.5), delta ~ U[0.8, 1.2), drawn in that order; the kernel's
    arguments are (a, b, c, d) = (alpha, beta, delta, gamma)."""
    rng = np.random.default_rng(seed)
    x0 = rng.uniform(0.5, 2.0, n).astype(np.float32)
    y0 = rng.uniform(0.5, 2.0, n).astype(np.float32)
    alpha = rng.uniform(0.8, 1.2, n).astype(np.float32)
    beta = rng.uniform(0.3, 0.5, n).astype(np.float32)
    gamma = rng.uniform(2.5, 3.5, n).astype(np.float32)
    delta = rng.uniform(0.8, 1.2, n).astype(np.float32)
    return x0, y0, alpha, beta, delta, gamma


def van_der_pol_ensemble(n: int, seed: int = 3):
    """(x0, v0, mu): mu log-uniform on [0.1, 10], x0, v0 ~ U[-2, 2)."""
    rng = np.random.default_rng(seed)
    mu = np.exp(rng.uniform(np.log(0.1), np.log(10.0), n)).astype(np.float32)
    x0 = rng.uniform(-2.0, 2.0, n).astype(np.float32)
    v0 = rng.uniform(-2.0, 2.0, n).astype(np.float32)
    return x0, v0, mu


def gbm_key(seed: int = 0) -> np.ndarray:
    """Threefry key data for an integer seed: (high word, low word)."""
    return np.array([(seed >> 32) & 0xFFFFFFFF, seed & 0xFFFFFFFF], dtype=np.uint32)


def gray_scott_initial_state(size: int, seed: int = 11, patches: int = 64, patch: int = 32):
    """u = 1, v = 0; `patches` square patches (periodic wrap) of u = 0.5,
    v = 0.25 at seeded top-left corners; then U[0, 0.01) noise on u."""
    rng = np.random.default_rng(seed)
    u = np.ones((size, size), np.float32)
    v = np.zeros((size, size), np.float32)
    corners = rng.integers(0, size, size=(patches, 2))
    span = np.arange(min(patch, size))
    for r, c in corners:
        rows = (r + span) % size
        cols = (c + span) % size
        u[np.ix_(rows, cols)] = 0.5
        v[np.ix_(rows, cols)] = 0.25
    u += rng.uniform(0.0, 0.01, (size, size)).astype(np.float32)
    return u, v


def split_df32(value) -> tuple[np.ndarray, np.ndarray]:
    """float64 -> (hi, lo) float32 pair with hi + lo == value to ~2^-48."""
    value = np.asarray(value, np.float64)
    hi = value.astype(np.float32)
    lo = (value - hi.astype(np.float64)).astype(np.float32)
    return hi, lo


def join_df32(hi, lo) -> np.ndarray:
    return np.asarray(hi, np.float64) + np.asarray(lo, np.float64)


def kepler_ensemble(n: int, seed: int = 5):
    """Two-body orbits, GM = 1: eccentricity ~ U[0, 0.7), semi-major axis
    ~ U[0.5, 2), true anomaly ~ U[0, 2 pi).  Returns the float64 state
    (N, 4) = (x, y, vx, vy) and the same state as eight float32 arrays
    (x_hi, x_lo, y_hi, y_lo, vx_hi, vx_lo, vy_hi, vy_lo).  The float64 state
    is rebuilt from the pairs so both start from identical numbers."""
    rng = np.random.default_rng(seed)
    e = rng.uniform(0.0, 0.7, n)
    a = rng.uniform(0.5, 2.0, n)
    theta = rng.uniform(0.0, 2.0 * np.pi, n)
    p = a * (1.0 - e * e)
    r = p / (1.0 + e * np.cos(theta))
    h = np.sqrt(p)
    comps = (r * np.cos(theta), r * np.sin(theta), -np.sin(theta) / h, (e + np.cos(theta)) / h)
    pairs = []
    for comp in comps:
        hi, lo = split_df32(comp)
        pairs += [hi, lo]
    state64 = np.stack([join_df32(pairs[2 * i], pairs[2 * i + 1]) for i in range(4)], axis=1)
    return state64, tuple(pairs)


def kepler_energy(state: np.ndarray, gm: float = 1.0) -> np.ndarray:
    """Specific orbital energy E = |v|^2 / 2 - GM / |r| of (N, 4) float64 states."""
    state = np.asarray(state, np.float64)
    r = np.hypot(state[:, 0], state[:, 1])
    return 0.5 * (state[:, 2] ** 2 + state[:, 3] ** 2) - gm / r
