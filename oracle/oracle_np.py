"""NumPy restatement of the reference kernels.  TEST INFRASTRUCTURE ONLY.

A second, independent statement of the same algorithms as `oracle.c`, vectorised
over the ensemble; the CPU tests require the two to agree bit for bit wherever
the arithmetic is IEEE-exact (integer hashing, +, -, *, /), which guards each
against transcription slips in the other.  NumPy float32 scalars and arrays
follow IEEE binary32; Python floats are folded in double and rounded once on
contact with a float32 array (NEP 50), the same rule JAX's weak types follow.
"""

from __future__ import annotations

import numpy as np

U32 = np.uint32
F32 = np.float32

_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))
# (rotation set, ks index for x0, ks index for x1, counter)  src/palladium/emit/rules.py:152-163
_SCHEDULE = ((0, 1, 2, 1), (1, 2, 0, 2), (0, 0, 1, 3), (1, 1, 2, 4), (0, 2, 0, 5))


def threefry2x32(k1, k2, c_hi, c_lo):
    """Threefry-2x32-20 on uint32 arrays (src/palladium/emit/rules.py:121-165)."""
    with np.errstate(over="ignore"):
        k1, k2 = np.asarray(k1, U32), np.asarray(k2, U32)
        ks = (k1, k2, k1 ^ k2 ^ U32(0x1BD11BDA))
        x0 = np.asarray(c_hi, U32) + ks[0]
        x1 = np.asarray(c_lo, U32) + ks[1]
        for rot_set, a, b, n in _SCHEDULE:
            for r in _ROT[rot_set]:
                x0 = x0 + x1
                x1 = (x1 << U32(r)) | (x1 >> U32(32 - r))
                x1 = x0 ^ x1
            x0 = x0 + ks[a]
            x1 = x1 + ks[b] + U32(n)
    return x0, x1


def random_bits(key, n: int) -> np.ndarray:
    x0, x1 = threefry2x32(key[0], key[1], U32(0), np.arange(n, dtype=U32))
    return x0 ^ x1


def bits_to_uniform(bits: np.ndarray) -> np.ndarray:
    return ((bits >> U32(9)) | U32(0x3F800000)).view(F32) - F32(1.0)


def uniform(key, n: int) -> np.ndarray:
    return bits_to_uniform(random_bits(key, n))


def fold_in(key, data) -> np.ndarray:
    x0, x1 = threefry2x32(key[0], key[1], U32(0), np.asarray(data, U32))
    return np.stack([x0, x1], axis=-1)


def lv_rk4(x0, y0, a, b, c, d, *, dt: float, steps: int):
    """examples/01_ode_ensembles.py:72-91, float32, staged op order."""
    x, y = np.asarray(x0, F32).copy(), np.asarray(y0, F32).copy()
    a, b, c, d = (np.asarray(v, F32) for v in (a, b, c, d))
    hh, hf, h6 = F32(0.5 * dt), F32(dt), F32(dt / 6.0)
    two = F32(2.0)

    def rhs(x, y):
        return a * x - b * x * y, c * x * y - d * y

    for _ in range(steps):
        k1x, k1y = rhs(x, y)
        k2x, k2y = rhs(x + hh * k1x, y + hh * k1y)
        k3x, k3y = rhs(x + hh * k2x, y + hh * k2y)
        k4x, k4y = rhs(x + hf * k3x, y + hf * k3y)
        x, y = (x + h6 * (k1x + two * k2x + two * k3x + k4x),
                y + h6 * (k1y + two * k2y + two * k3y + k4y))
    return x, y


def gray_scott(u, v, *, steps: int, du=0.16, dv=0.08, f=0.035, k=0.065, dt=1.0):
    """examples/04_reaction_diffusion.py:61-74 applied to every cell, periodic."""
    u, v = np.asarray(u, F32).copy(), np.asarray(v, F32).copy()
    DU, DV, F, FK, DT = F32(du), F32(dv), F32(f), F32(f + k), F32(dt)
    four, one = F32(4.0), F32(1.0)
    rows, cols = u.shape
    ip = np.r_[1:rows, 0]
    im = np.r_[rows - 1, 0:rows - 1]
    jp = np.r_[1:cols, 0]
    jm = np.r_[cols - 1, 0:cols - 1]
    for _ in range(steps):
        lap_u = u[ip, :] + u[im, :] + u[:, jp] + u[:, jm] - four * u
        lap_v = v[ip, :] + v[im, :] + v[:, jp] + v[:, jm] - four * v
        uvv = u * v * v
        u, v = (u + DT * (DU * lap_u - uvv + F * (one - u)),
                v + DT * (DV * lap_v + uvv - FK * v))
    return u, v


def gray_scott_slab(u, v, *, steps: int, halo: int, du=0.16, dv=0.08, f=0.035, k=0.065, dt=1.0):
    """The same stencil on a row slab with `halo` ghost rows above and below:
    periodic in columns only; step s (1-based) updates rows [s, rows_alloc - s)
    and leaves the others as they were."""
    u, v = np.asarray(u, F32).copy(), np.asarray(v, F32).copy()
    if steps > halo:
        raise ValueError("a slab can advance at most `halo` steps between exchanges")
    DU, DV, F, FK, DT = F32(du), F32(dv), F32(f), F32(f + k), F32(dt)
    four, one = F32(4.0), F32(1.0)
    rows, cols = u.shape
    jp = np.r_[1:cols, 0]
    jm = np.r_[cols - 1, 0:cols - 1]
    for s in range(1, steps + 1):
        lo, hi = s, rows - s
        uc, vc = u[lo:hi], v[lo:hi]
        lap_u = u[lo + 1:hi + 1] + u[lo - 1:hi - 1] + uc[:, jp] + uc[:, jm] - four * uc
        lap_v = v[lo + 1:hi + 1] + v[lo - 1:hi - 1] + vc[:, jp] + vc[:, jm] - four * vc
        uvv = uc * vc * vc
        nu = uc + DT * (DU * lap_u - uvv + F * (one - uc))
        nv = vc + DT * (DV * lap_v + uvv - FK * vc)
        u, v = u.copy(), v.copy()
        u[lo:hi], v[lo:hi] = nu, nv
    return u, v


def gbm(key, n: int, *, s0, strike, r, sigma, t, steps: int, path_offset: int = 0):
    """examples/03_sde_montecarlo.py:97-119 with NumPy's float32 log/cos/exp,
    which are not the C library's: agreement with oracle.c is to rounding
    error, not bit for bit."""
    key = np.asarray(key, U32)
    dt = t / steps
    drift_dt = F32((r - sigma**2 / 2) * dt)
    vol_sqdt = F32(sigma) * np.sqrt(F32(dt))
    two_pi = F32(2.0 * np.pi)
    key0 = fold_in(key, np.arange(path_offset, path_offset + n, dtype=np.uint64).astype(U32))
    s = np.full(n, s0, F32)
    for i in range(steps):
        ka = threefry2x32(key0[:, 0], key0[:, 1], U32(0), U32(2 * i))
        kb = threefry2x32(key0[:, 0], key0[:, 1], U32(0), U32(2 * i + 1))
        ba = threefry2x32(ka[0], ka[1], U32(0), U32(0))
        bb = threefry2x32(kb[0], kb[1], U32(0), U32(0))
        u1 = np.maximum(bits_to_uniform(ba[0] ^ ba[1]), F32(1e-7))
        u2 = bits_to_uniform(bb[0] ^ bb[1])
        z = np.sqrt(F32(-2.0) * np.log(u1)) * np.cos(two_pi * u2)
        s = s * np.exp(drift_dt + vol_sqdt * z)
    return s, np.maximum(s - F32(strike), F32(0.0))


def pcg_hash(v) -> np.ndarray:
    """examples/03_sde_montecarlo.py:38-43 on uint32 arrays."""
    with np.errstate(over="ignore"):
        v = np.asarray(v, U32)
        state = v * U32(747796405) + U32(2891336453)
        word = ((state >> ((state >> U32(28)) + U32(4))) ^ state) * U32(277803737)
        return (word >> U32(22)) ^ word


def pcg_uniform01(v) -> np.ndarray:
    return (pcg_hash(v).astype(F32) + F32(0.5)) * F32(2.3283064e-10)
