"""CPU oracle for `families.custom_ode`.  TEST INFRASTRUCTURE ONLY.

Builds `custom_ode_template.c` around a right-hand side (the same text the CUDA
library hands to NVRTC; it has to be valid C as well as CUDA C) with
`gcc -O2 -ffp-contract=off`, one shared object per (source, dim, nparam) under
`oracle/_custom/`, and calls it through ctypes.
"""

from __future__ import annotations

import ctypes
import hashlib
import subprocess
from pathlib import Path

import numpy as np

from . import build as _build

_HERE = Path(__file__).resolve().parent
_OUT = _HERE / "_custom"
_TEMPLATE = _HERE / "custom_ode_template.c"
_HEADER_DIR = _HERE.parent / "palladium_b200" / "csrc"
_libs: dict = {}

BS32_DEFAULTS = dict(t1=10.0, rtol=1e-5, atol=1e-7, dt0=0.01, pcoeff=0.4, icoeff=0.3, safety=0.9, factor_min=0.2,
                     factor_max=10.0, error_order=3, max_steps=6000)


def _lib(rhs: str, dim: int, nparam: int) -> ctypes.CDLL:
    key = (rhs, dim, nparam)
    if key in _libs:
        return _libs[key]
    template = _TEMPLATE.read_text()
    digest = hashlib.sha256(f"{dim}|{nparam}|{rhs}|{template}".encode()).hexdigest()[:16]
    _OUT.mkdir(exist_ok=True)
    src, lib = _OUT / f"ode_{digest}.c", _OUT / f"ode_{digest}.so"
    if not lib.exists():
        src.write_text(template.replace("/*ORC_RHS*/", rhs))
        cmd = ["gcc", "-std=c11", *_build.CFLAGS, f"-I{_HEADER_DIR}", f"-DORC_DIM={dim}", f"-DORC_NPARAM={nparam}",
               f"-DORC_NPARAM_ALLOC={max(nparam, 1)}", str(src), "-o", str(lib), "-lm"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"oracle build of a custom right-hand side failed:\n{proc.stderr}")
    _libs[key] = ctypes.CDLL(str(lib))
    return _libs[key]


def _pointers(arrays):
    fp = ctypes.POINTER(ctypes.c_float)
    return (fp * max(len(arrays), 1))(*[a.ctypes.data_as(fp) for a in arrays])


def rk4(rhs: str, dim: int, nparam: int, arrays, *, dt: float, steps: int):
    """`dim` final-state arrays after `steps` RK4 steps of `dt`."""
    ins = [np.ascontiguousarray(a, np.float32) for a in arrays]
    assert len(ins) == dim + nparam
    n = ins[0].size
    outs = [np.empty(n, np.float32) for _ in range(dim)]
    fn = _lib(rhs, dim, nparam).orc_custom_rk4
    fn.restype = None
    fn(ctypes.c_int64(n), _pointers(ins), _pointers(outs), ctypes.c_int64(steps), ctypes.c_double(dt))
    return tuple(outs)


def bs32(rhs: str, dim: int, nparam: int, arrays, *, pow: str = "libm", **params):
    """(t, states..., steps, rejected, real) of the adaptive loop."""
    cfg = dict(BS32_DEFAULTS)
    cfg.update(params)
    ins = [np.ascontiguousarray(a, np.float32) for a in arrays]
    assert len(ins) == dim + nparam
    n = ins[0].size
    outs = [np.empty(n, np.float32) for _ in range(dim + 4)]
    fn = _lib(rhs, dim, nparam).orc_custom_bs32
    fn.restype = None
    d = ctypes.c_double
    fn(ctypes.c_int64(n), _pointers(ins), _pointers(outs), d(cfg["t1"]), d(cfg["rtol"]), d(cfg["atol"]),
       d(cfg["dt0"]), d(cfg["pcoeff"]), d(cfg["icoeff"]), d(cfg["safety"]), d(cfg["factor_min"]),
       d(cfg["factor_max"]), ctypes.c_int64(cfg["error_order"]), ctypes.c_int64(cfg["max_steps"]),
       ctypes.c_int({"libm": 0, "pd": 1}[pow]))
    return tuple(outs)


ERK_METHODS = {"dopri5": 2, "tsit5": 3}


def erk(rhs: str, dim: int, nparam: int, arrays, *, method: str, pow: str = "libm", **params):
    """(t, states..., steps, rejected, real) of the adaptive loop around a seven-stage 5(4) pair
    ("dopri5" or "tsit5"); `error_order` defaults to 5."""
    cfg = dict(BS32_DEFAULTS, error_order=5)
    cfg.update(params)
    ins = [np.ascontiguousarray(a, np.float32) for a in arrays]
    assert len(ins) == dim + nparam
    n = ins[0].size
    outs = [np.empty(n, np.float32) for _ in range(dim + 4)]
    fn = _lib(rhs, dim, nparam).orc_custom_erk
    fn.restype = None
    d = ctypes.c_double
    fn(ctypes.c_int64(n), _pointers(ins), _pointers(outs), ctypes.c_int(ERK_METHODS[method]), d(cfg["t1"]),
       d(cfg["rtol"]), d(cfg["atol"]), d(cfg["dt0"]), d(cfg["pcoeff"]), d(cfg["icoeff"]), d(cfg["safety"]),
       d(cfg["factor_min"]), d(cfg["factor_max"]), ctypes.c_int64(cfg["error_order"]),
       ctypes.c_int64(cfg["max_steps"]), ctypes.c_int({"libm": 0, "pd": 1}[pow]))
    return tuple(outs)


def tableau(method: str):
    """(A, c, e) of a 5(4) pair as float64 arrays, read back from the coefficients the compiled
    oracle holds (float32 values): A is 7 x 7 strictly lower triangular with the weights as its
    last row."""
    lib = _lib("dy[0] = y[0];", 1, 0)
    fn = lib.orc_tableau
    fn.restype = None
    a = np.zeros((6, 6), np.float32)
    c = np.zeros(7, np.float32)
    e = np.zeros(7, np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    fn(ctypes.c_int(ERK_METHODS[method]), a.ctypes.data_as(fp), c.ctypes.data_as(fp), e.ctypes.data_as(fp))
    full = np.zeros((7, 7))
    full[1:, :6] = a
    return full, c.astype(np.float64), e.astype(np.float64)
