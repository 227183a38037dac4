"""CPU oracle for the ensemble-integrator kernels.  TEST INFRASTRUCTURE ONLY.

Only `tests/`, the smoke check and the CPU-baseline leg of the benchmark may
import this package; the shipped package (`palladium_b200`) never does.

It stands in for the reference's `call.interpret(*args)` (the Pallas CPU
interpreter, src/palladium/__init__.py:110), which needs JAX.  Two independent
restatements live here: `oracle.c` (C, OpenMP; bound below through ctypes) and
`oracle_np.py` (NumPy).  See the header of `oracle.c` for what each kernel
follows in the reference and for which parts have a pin and which are
"parity unpinned".
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

from . import build as _build
from . import oracle_np  # noqa: F401  (re-exported for tests)

_HERE = Path(__file__).resolve().parent
_lib = None
_ref = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_i64 = ctypes.c_int64
_dbl = ctypes.c_double


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.ORACLE_LIB
        if not path.exists():
            _build.build_oracle()
        _lib = ctypes.CDLL(str(path))
        _lib.orc_max_threads.restype = ctypes.c_int
    return _lib


def reference_lib() -> ctypes.CDLL | None:
    """The reference's own golden RK4 kernel compiled for the CPU, or None when
    it has not been built (it can only be built next to a reference checkout)."""
    global _ref
    if _ref is None and _build.REF_LIB.exists():
        _ref = ctypes.CDLL(str(_build.REF_LIB))
    return _ref


_ref_threefry = None


def reference_threefry_lib() -> ctypes.CDLL | None:
    """The Threefry block as the reference's emitter writes it, compiled for the
    CPU, or None when it has not been built (needs a reference checkout)."""
    global _ref_threefry
    if _ref_threefry is None and _build.REF_THREEFRY_LIB.exists():
        _ref_threefry = ctypes.CDLL(str(_build.REF_THREEFRY_LIB))
    return _ref_threefry


def reference_threefry(key, counters) -> np.ndarray:
    """Blocks (key, counters[i]) -> (n, 2) uint32 through the reference's emitted statements."""
    ref = reference_threefry_lib()
    if ref is None:
        raise RuntimeError("oracle/_ref/libthreefryref.so is not built")
    key = _u32(key)
    counters = _u32(counters).reshape(-1, 2)
    out = np.empty_like(counters)
    for i in range(counters.shape[0]):
        ref.ref_threefry2x32(_p(key, _u32p), _p(counters[i].copy(), _u32p), _p(out[i:i + 1], _u32p))
    return out


def reference_random_bits(key, n: int) -> np.ndarray:
    ref = reference_threefry_lib()
    if ref is None:
        raise RuntimeError("oracle/_ref/libthreefryref.so is not built")
    key = _u32(key)
    out = np.empty(n, np.uint32)
    ref.ref_random_bits(_p(key, _u32p), ctypes.c_longlong(n), _p(out, _u32p))
    return out


def reference_fold_in(key, data) -> np.ndarray:
    ref = reference_threefry_lib()
    if ref is None:
        raise RuntimeError("oracle/_ref/libthreefryref.so is not built")
    key, data = _u32(key), _u32(np.atleast_1d(data))
    out = np.empty((data.size, 2), np.uint32)
    ref.ref_fold_in(_p(key, _u32p), _p(data, _u32p), ctypes.c_longlong(data.size), _p(out, _u32p))
    return out


_ref_gbm = None


def reference_gbm_lib() -> ctypes.CDLL | None:
    """The reference's hand-written `gbm_paths` MSL kernel compiled for the CPU,
    or None when it has not been built (needs a reference checkout)."""
    global _ref_gbm
    if _ref_gbm is None and _build.REF_GBM_LIB.exists():
        _ref_gbm = ctypes.CDLL(str(_build.REF_GBM_LIB))
    return _ref_gbm


def reference_gbm_paths(n: int, *, s0: float, strike: float, r: float, sigma: float, t: float, steps: int):
    """Payoffs of the reference's own kernel, scalars formed as its driver forms
    them (examples/03_sde_montecarlo.py:80-89)."""
    ref = reference_gbm_lib()
    if ref is None:
        raise RuntimeError("oracle/_ref/libgbmref.so is not built")
    dt = t / steps
    drift_dt = np.float32((r - sigma**2 / 2) * dt)
    vol_sqdt = np.float32(sigma * np.sqrt(dt))
    payoff = np.empty(n, np.float32)
    ref.ref_gbm_paths(_i64(n), ctypes.c_uint32(steps), ctypes.c_float(s0), ctypes.c_float(strike),
                      ctypes.c_float(float(drift_dt)), ctypes.c_float(float(vol_sqdt)), _p(payoff, _f32p))
    return payoff


def reference_pcg_hash(values) -> np.ndarray:
    ref = reference_gbm_lib()
    if ref is None:
        raise RuntimeError("oracle/_ref/libgbmref.so is not built")
    values = _u32(values)
    out = np.empty_like(values)
    ref.ref_pcg_hash(_i64(values.size), _p(values, _u32p), _p(out, _u32p))
    return out


_ref_df32 = None


def reference_lv_rk4_df32(x0, y0, a, b, c, d, *, dt: float, steps: int):
    """The reference's own df32 kernel text (examples/05_df32_precision.py:27-80)
    on this oracle's df32 prelude; scalars as its driver passes them (:158)."""
    global _ref_df32
    if _ref_df32 is None:
        if not _build.REF_DF32_LIB.exists():
            raise RuntimeError("oracle/_ref/libdf32ref.so is not built")
        _ref_df32 = ctypes.CDLL(str(_build.REF_DF32_LIB))
    arrs = [_f32(v) for v in (x0, y0, a, b, c, d)]
    n = arrs[0].size
    xo, yo = np.empty(n, np.float32), np.empty(n, np.float32)
    _ref_df32.ref_lv_rk4_df32(_i64(n), *[_p(v, _f32p) for v in arrs], _p(xo, _f32p), _p(yo, _f32p),
                              ctypes.c_float(float(np.float32(dt))), ctypes.c_uint32(steps))
    return xo, yo


def libm_f32(op: str, x, y=None) -> np.ndarray:
    """powf / expf / logf / cosf / sqrtf of the C library, elementwise on float32."""
    code = {"pow": 0, "exp": 1, "log": 2, "cos": 3, "sqrt": 4}[op]
    x = np.ascontiguousarray(x, np.float32)
    shape = x.shape
    x = x.reshape(-1)
    y = x if y is None else np.ascontiguousarray(np.broadcast_to(np.asarray(y, np.float32), shape)).reshape(-1)
    out = np.empty_like(x)
    lib().orc_libm_f32(ctypes.c_int(code), _i64(x.size), _p(x, _f32p), _p(y, _f32p), _p(out, _f32p))
    return out.reshape(shape)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def set_threads(n: int) -> None:
    lib().orc_set_threads(ctypes.c_int(int(n)))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _p(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


# --------------------------------------------------------------------------- RNG
def threefry2x32(key, ctr) -> np.ndarray:
    key, ctr = _u32(key), _u32(ctr)
    out = np.empty(2, np.uint32)
    lib().orc_threefry2x32(_p(key, _u32p), _p(ctr, _u32p), _p(out, _u32p))
    return out


def random_bits(key, n: int) -> np.ndarray:
    key = _u32(key)
    out = np.empty(n, np.uint32)
    lib().orc_random_bits(_p(key, _u32p), _i64(n), _p(out, _u32p))
    return out


def uniform(key, n: int) -> np.ndarray:
    key = _u32(key)
    out = np.empty(n, np.float32)
    lib().orc_uniform(_p(key, _u32p), _i64(n), _p(out, _f32p))
    return out


def fold_in(key, data) -> np.ndarray:
    key, data = _u32(key), _u32(np.atleast_1d(data))
    out = np.empty((data.size, 2), np.uint32)
    lib().orc_fold_in(_p(key, _u32p), _p(data, _u32p), _i64(data.size), _p(out, _u32p))
    return out


def fold_uniform(key, groups: int, count: int) -> np.ndarray:
    key = _u32(key)
    out = np.empty((groups, count), np.float32)
    lib().orc_fold_uniform(_p(key, _u32p), _i64(groups), _i64(count), _p(out, _f32p))
    return out


# --------------------------------------------------------------------------- RK4 LV
def lv_rk4(x0, y0, a, b, c, d, *, dt: float, steps: int):
    arrs = [_f32(v) for v in (x0, y0, a, b, c, d)]
    n = arrs[0].size
    xo, yo = np.empty(n, np.float32), np.empty(n, np.float32)
    lib().orc_lv_rk4(_i64(n), *[_p(v, _f32p) for v in arrs], _p(xo, _f32p), _p(yo, _f32p), _dbl(dt), _i64(steps))
    return xo, yo


def lv_rk4_f64(x0, y0, a, b, c, d, *, dt: float, steps: int):
    arrs = [_f32(v) for v in (x0, y0, a, b, c, d)]
    n = arrs[0].size
    xo, yo = np.empty(n, np.float64), np.empty(n, np.float64)
    lib().orc_lv_rk4_f64(_i64(n), *[_p(v, _f32p) for v in arrs], _p(xo, _f64p), _p(yo, _f64p), _dbl(dt), _i64(steps))
    return xo, yo


def lv_rk4_reference_golden(x0, y0, a, b, c, d):
    """The reference's emitted kernel itself (500 steps of dt = 0.01)."""
    ref = reference_lib()
    if ref is None:
        raise RuntimeError("oracle/_ref/libmslref.so is not built")
    arrs = [_f32(v) for v in (x0, y0, a, b, c, d)]
    n = arrs[0].size
    xo, yo = np.empty(n, np.float32), np.empty(n, np.float32)
    ref.ref_rk4_lv_golden(_i64(n), *[_p(v, _f32p) for v in arrs], _p(xo, _f32p), _p(yo, _f32p))
    return xo, yo


# --------------------------------------------------------------------------- adaptive
VDP_DEFAULTS = dict(t1=10.0, rtol=1e-5, atol=1e-7, dt0=0.01, pcoeff=0.4, icoeff=0.3, safety=0.9,
                    factor_min=0.2, factor_max=10.0, error_order=3, max_steps=6000)


def vdp_bs32(x0, v0, mu, *, pow: str = "libm", **params):
    """Returns (t, x, v, steps, rejected, real), six float32 arrays."""
    cfg = dict(VDP_DEFAULTS)
    cfg.update(params)
    x0, v0, mu = _f32(x0), _f32(v0), _f32(mu)
    n = x0.size
    outs = [np.empty(n, np.float32) for _ in range(6)]
    lib().orc_vdp_bs32(
        _i64(n), _p(x0, _f32p), _p(v0, _f32p), _p(mu, _f32p), *[_p(o, _f32p) for o in outs],
        _dbl(cfg["t1"]), _dbl(cfg["rtol"]), _dbl(cfg["atol"]), _dbl(cfg["dt0"]), _dbl(cfg["pcoeff"]),
        _dbl(cfg["icoeff"]), _dbl(cfg["safety"]), _dbl(cfg["factor_min"]), _dbl(cfg["factor_max"]),
        _i64(cfg["error_order"]), _i64(cfg["max_steps"]), ctypes.c_int({"libm": 0, "pd": 1}[pow]))
    return tuple(outs)


# --------------------------------------------------------------------------- GBM
def gbm_constants(r: float, sigma: float, t: float, steps: int):
    """drift_dt and vol_sqdt as the kernel body forms them (examples/03:98-100):
    the drift folds in double and rounds once; the volatility term is
    f32(sigma) * sqrt_f32(f32(dt))."""
    dt = t / steps
    drift_dt = np.float32((r - sigma**2 / 2) * dt)
    vol_sqdt = np.float32(sigma) * np.sqrt(np.float32(dt))
    return drift_dt, np.float32(vol_sqdt)


def gbm(key, n: int, *, s0: float, strike: float, r: float, sigma: float, t: float, steps: int,
        path_offset: int = 0):
    """Returns (terminal price, payoff), float32 arrays of n paths."""
    key = _u32(key)
    drift_dt, vol_sqdt = gbm_constants(r, sigma, t, steps)
    terminal, payoff = np.empty(n, np.float32), np.empty(n, np.float32)
    lib().orc_gbm(_i64(n), _p(key, _u32p), _i64(path_offset), _i64(steps), ctypes.c_float(s0),
                  ctypes.c_float(strike), ctypes.c_float(float(drift_dt)), ctypes.c_float(float(vol_sqdt)),
                  _p(terminal, _f32p), _p(payoff, _f32p))
    return terminal, payoff


def pcg_hash(n: int) -> np.ndarray:
    out = np.empty(n, np.uint32)
    lib().orc_pcg_hash(_i64(n), _p(out, _u32p))
    return out


def gbm_pcg(n: int, *, s0: float, strike: float, r: float, sigma: float, t: float, steps: int, path_offset: int = 0):
    """The hand-written kernel's paths; scalars as `run_handwritten` forms them
    (examples/03_sde_montecarlo.py:80-89).  Returns (terminal, payoff)."""
    dt = t / steps
    drift_dt = np.float32((r - sigma**2 / 2) * dt)
    vol_sqdt = np.float32(sigma * np.sqrt(dt))
    terminal, payoff = np.empty(n, np.float32), np.empty(n, np.float32)
    lib().orc_gbm_pcg(_i64(n), _i64(path_offset), _i64(steps), ctypes.c_float(s0), ctypes.c_float(strike),
                      ctypes.c_float(float(drift_dt)), ctypes.c_float(float(vol_sqdt)), _p(terminal, _f32p),
                      _p(payoff, _f32p))
    return terminal, payoff


def black_scholes_call(s0: float, k: float, t: float, r: float, sigma: float) -> float:
    """Closed form the Monte Carlo price is checked against (examples/03:73-76)."""
    from math import erf, exp, log, sqrt

    def cdf(x):
        return 0.5 * (1.0 + erf(x / sqrt(2.0)))

    d1 = (log(s0 / k) + (r + sigma**2 / 2) * t) / (sigma * sqrt(t))
    d2 = d1 - sigma * sqrt(t)
    return s0 * cdf(d1) - k * exp(-r * t) * cdf(d2)


# --------------------------------------------------------------------------- Gray-Scott
GS_DEFAULTS = dict(du=0.16, dv=0.08, f=0.035, k=0.065, dt=1.0)


def gray_scott(u, v, *, steps: int, **params):
    cfg = dict(GS_DEFAULTS)
    cfg.update(params)
    u, v = _f32(u), _f32(v)
    rows, cols = u.shape
    uo, vo = np.empty_like(u), np.empty_like(v)
    rc = lib().orc_gray_scott(_i64(rows), _i64(cols), _p(u, _f32p), _p(v, _f32p), _p(uo, _f32p), _p(vo, _f32p),
                              _dbl(cfg["du"]), _dbl(cfg["dv"]), _dbl(cfg["f"]), _dbl(cfg["k"]), _dbl(cfg["dt"]),
                              _i64(steps))
    if rc:
        raise MemoryError("oracle gray_scott: allocation failed")
    return uo, vo


# --------------------------------------------------------------------------- df32
def df_op(op: str, a_hi, a_lo, b_hi=None, b_lo=None):
    code = {"add": 0, "sub": 1, "mul": 2, "div": 3, "sqrt": 4, "recip": 5, "rsqrt": 6}[op]
    a_hi, a_lo = _f32(a_hi), _f32(a_lo)
    b_hi = _f32(b_hi) if b_hi is not None else np.ones_like(a_hi)
    b_lo = _f32(b_lo) if b_lo is not None else np.zeros_like(a_hi)
    oh, ol = np.empty_like(a_hi), np.empty_like(a_hi)
    lib().orc_df_op(ctypes.c_int(code), _i64(a_hi.size), _p(a_hi, _f32p), _p(a_lo, _f32p), _p(b_hi, _f32p),
                    _p(b_lo, _f32p), _p(oh, _f32p), _p(ol, _f32p))
    return oh, ol


def eft(op: str, a, b):
    code = {"two_sum": 0, "two_prod": 1}[op]
    a, b = _f32(a), _f32(b)
    hi, lo = np.empty_like(a), np.empty_like(a)
    lib().orc_eft(ctypes.c_int(code), _i64(a.size), _p(a, _f32p), _p(b, _f32p), _p(hi, _f32p), _p(lo, _f32p))
    return hi, lo


def lv_rk4_df32(x0, y0, a, b, c, d, *, dt: float, steps: int):
    arrs = [_f32(v) for v in (x0, y0, a, b, c, d)]
    n = arrs[0].size
    xo, yo = np.empty(n, np.float32), np.empty(n, np.float32)
    lib().orc_lv_rk4_df32(_i64(n), *[_p(v, _f32p) for v in arrs], _p(xo, _f32p), _p(yo, _f32p), _dbl(dt),
                          _i64(steps))
    return xo, yo


def kepler_rk4_df32(state8, *, dt: float, gm: float = 1.0, steps: int):
    """state8: eight float32 arrays (x_hi, x_lo, y_hi, y_lo, vx_hi, vx_lo, vy_hi, vy_lo)."""
    ins = [_f32(v) for v in state8]
    n = ins[0].size
    outs = [np.empty(n, np.float32) for _ in range(8)]
    in_ptrs = (_f32p * 8)(*[_p(v, _f32p) for v in ins])
    out_ptrs = (_f32p * 8)(*[_p(v, _f32p) for v in outs])
    lib().orc_kepler_rk4_df32(_i64(n), in_ptrs, out_ptrs, _dbl(dt), _dbl(gm), _i64(steps))
    return tuple(outs)


def kepler_rk4_f64(state, *, dt: float, gm: float = 1.0, steps: int) -> np.ndarray:
    """state: (N, 4) float64 rows (x, y, vx, vy)."""
    state = np.ascontiguousarray(state, dtype=np.float64)
    out = np.empty_like(state)
    lib().orc_kepler_rk4_f64(_i64(state.shape[0]), _p(state, _f64p), _p(out, _f64p), _dbl(dt), _dbl(gm), _i64(steps))
    return out


def kepler_rk4_f32(state, *, dt: float, gm: float = 1.0, steps: int) -> np.ndarray:
    state = np.ascontiguousarray(state, dtype=np.float32)
    out = np.empty_like(state)
    lib().orc_kepler_rk4_f32(_i64(state.shape[0]), _p(state, _f32p), _p(out, _f32p), _dbl(dt), _dbl(gm), _i64(steps))
    return out


def pd_ctrl_pow(err, c) -> np.ndarray:
    """(1 / err) ** c through the float routine the adaptive kernels' step controller uses."""
    err, c = _f32(err), _f32(c)
    err, c = np.broadcast_arrays(err, c)
    err, c = np.ascontiguousarray(err), np.ascontiguousarray(c)
    out = np.empty_like(err)
    lib().orc_pd_ctrl_pow(_i64(err.size), _p(err, _f32p), _p(c, _f32p), _p(out, _f32p))
    return out


def pd_powf(x, y) -> np.ndarray:
    x, y = _f32(x), _f32(y)
    x, y = np.broadcast_arrays(x, y)
    x, y = np.ascontiguousarray(x), np.ascontiguousarray(y)
    out = np.empty_like(x)
    lib().orc_pd_powf(_i64(x.size), _p(x, _f32p), _p(y, _f32p), _p(out, _f32p))
    return out
