"""ctypes binding of libpalladium_cuda.so (declared in include/palladium_cuda.h).

This is the Python half of the drop-in boundary: the reference loads its native
handler with `ctypes.CDLL` and hands it to XLA (src/palladium/ffi.py:64-79);
here the same library is loaded the same way and its C entry points are called
directly.  `PALLADIUM_FFI_LIBRARY` overrides the path, as in the reference
(src/palladium/ffi.py:42).

There is no fallback: if the library is missing, every call raises EmitError
with the build command.
"""

from __future__ import annotations

import ctypes
import functools
import os
import threading
from pathlib import Path

from .errors import DispatchError, EmitError, PalladiumError

__all__ = [
    "library",
    "library_path",
    "LvRk4Params",
    "VdpBs32Params",
    "GbmParams",
    "GrayScottParams",
    "LvRk4Df32Params",
    "KeplerRk4Df32Params",
    "ThreefryParams",
    "LaunchInfo",
    "EXPORTED_SYMBOLS",
    "FAMILY_IDS",
]

_LIBRARY_NAME = "libpalladium_cuda.so"
PD_ABI_VERSION = 1

EXPORTED_SYMBOLS = (
    "pd_version",
    "pd_device_count",
    "pd_launch",
    "pd_dispatch_host",
    "pd_submit_host",
    "pd_wait_host",
    "pd_explain",
    "pd_set_tuning",
    "pd_get_tuning",
    "pd_set_thread_tuning",
    "pd_clear_thread_tuning",
    "pd_measure_fp32_fma_peak",
    "pd_measure_int32_alu_peak",
    "pd_last_kernel_ms",
    "pd_device_status",
    "pd_gray_scott_static",
    "pd_custom_ode_check",
    "pd_source_kernel_check",
    "pd_custom_ode_source",
    "pd_gray_scott_slab_push",
    "pd_peer_alloc",
    "pd_peer_export",
    "pd_peer_open",
    "pd_peer_close",
    "pd_peer_free",
)

FAMILY_IDS = {
    "lv_rk4": 0,
    "vdp_bs32": 1,
    "gbm_threefry": 2,
    "gray_scott": 3,
    "lv_rk4_df32": 4,
    "kepler_rk4_df32": 5,
    "threefry_bits": 6,
    "gbm_pcg": 7,
    "custom_ode": 8,
    "source": 9,
}

_i64 = ctypes.c_int64
_dbl = ctypes.c_double


class LvRk4Params(ctypes.Structure):
    _fields_ = [("dt", _dbl), ("steps", _i64)]


class VdpBs32Params(ctypes.Structure):
    _fields_ = [("t1", _dbl), ("rtol", _dbl), ("atol", _dbl), ("dt0", _dbl), ("pcoeff", _dbl), ("icoeff", _dbl),
                ("safety", _dbl), ("factor_min", _dbl), ("factor_max", _dbl), ("error_order", _i64),
                ("max_steps", _i64), ("out_layout", _i64)]


class GbmParams(ctypes.Structure):
    _fields_ = [("s0", _dbl), ("strike", _dbl), ("r", _dbl), ("sigma", _dbl), ("t", _dbl), ("steps", _i64),
                ("path_offset", _i64), ("output_kind", _i64)]


class GrayScottParams(ctypes.Structure):
    _fields_ = [("du", _dbl), ("dv", _dbl), ("f", _dbl), ("k", _dbl), ("dt", _dbl), ("steps", _i64),
                ("rows", _i64), ("cols", _i64), ("halo", _i64)]


class LvRk4Df32Params(ctypes.Structure):
    _fields_ = [("dt", _dbl), ("steps", _i64)]


class KeplerRk4Df32Params(ctypes.Structure):
    _fields_ = [("dt", _dbl), ("gm", _dbl), ("steps", _i64)]


class ThreefryParams(ctypes.Structure):
    _fields_ = [("op", _i64), ("count", _i64)]


class CustomOdeParams(ctypes.Structure):
    _fields_ = [("rhs_source", ctypes.c_char_p), ("dim", _i64), ("nparam", _i64), ("method", _i64), ("dt", _dbl),
                ("steps", _i64), ("t1", _dbl), ("rtol", _dbl), ("atol", _dbl), ("dt0", _dbl), ("pcoeff", _dbl),
                ("icoeff", _dbl), ("safety", _dbl), ("factor_min", _dbl), ("factor_max", _dbl),
                ("error_order", _i64), ("max_steps", _i64)]


class SourceKernelParams(ctypes.Structure):
    _fields_ = [("cuda_source", ctypes.c_char_p), ("function_name", ctypes.c_char_p)]


class GsNeighbours(ctypes.Structure):
    _fields_ = [("up_u", ctypes.c_void_p), ("up_v", ctypes.c_void_p), ("up_rows", _i64),
                ("down_u", ctypes.c_void_p), ("down_v", ctypes.c_void_p), ("down_rows", _i64)]


PEER_HANDLE_BYTES = 64


class LaunchInfo(ctypes.Structure):
    _fields_ = [("kernel_name", ctypes.c_char * 64), ("cuda_grid", _i64 * 3), ("cuda_block", _i64 * 3),
                ("items_per_thread", _i64), ("launches", _i64), ("scratch_bytes", _i64),
                ("regs_per_thread", ctypes.c_int32), ("static_smem_bytes", ctypes.c_int32),
                ("dynamic_smem_bytes", ctypes.c_int32), ("blocks_per_sm", ctypes.c_int32)]


def library_path() -> Path:
    override = os.environ.get("PALLADIUM_FFI_LIBRARY")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / _LIBRARY_NAME


_LOAD_LOCK = threading.Lock()
_lib: ctypes.CDLL | None = None


def _declare(lib: ctypes.CDLL) -> None:
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    i64p = ctypes.POINTER(_i64)
    vpp = ctypes.POINTER(vp)
    szp = ctypes.POINTER(sz)
    cp = ctypes.c_char_p
    lib.pd_version.restype = ci
    lib.pd_version.argtypes = []
    lib.pd_device_count.restype = ci
    lib.pd_device_count.argtypes = []
    lib.pd_launch.restype = ci
    lib.pd_launch.argtypes = [ci, vp, sz, ci, i64p, i64p, ci, vpp, szp, ci, vpp, szp, vp, sz, vp, cp, sz]
    lib.pd_dispatch_host.restype = ci
    lib.pd_dispatch_host.argtypes = [ci, vp, sz, ci, i64p, i64p, ci, vpp, szp, ci, vpp, szp, cp, sz]
    lib.pd_submit_host.restype = ci
    lib.pd_submit_host.argtypes = [ci, vp, sz, ci, i64p, i64p, ci, vpp, szp, ctypes.POINTER(ci), ci, vpp, szp, ctypes.POINTER(ctypes.c_uint64), cp, sz]
    lib.pd_wait_host.restype = ci
    lib.pd_wait_host.argtypes = [ctypes.c_uint64, ci, vpp, szp, cp, sz]
    lib.pd_explain.restype = ci
    lib.pd_explain.argtypes = [ci, vp, sz, ci, i64p, i64p, ctypes.POINTER(LaunchInfo), cp, sz]
    lib.pd_set_tuning.restype = ci
    lib.pd_set_tuning.argtypes = [cp, _i64]
    lib.pd_get_tuning.restype = ci
    lib.pd_get_tuning.argtypes = [cp, i64p]
    lib.pd_set_thread_tuning.restype = ci
    lib.pd_set_thread_tuning.argtypes = [cp, _i64]
    lib.pd_clear_thread_tuning.restype = ci
    lib.pd_clear_thread_tuning.argtypes = [cp]
    lib.pd_measure_fp32_fma_peak.restype = ci
    lib.pd_measure_fp32_fma_peak.argtypes = [ctypes.POINTER(_dbl), cp, sz]
    lib.pd_measure_int32_alu_peak.restype = ci
    lib.pd_measure_int32_alu_peak.argtypes = [ctypes.POINTER(_dbl), cp, sz]
    lib.pd_last_kernel_ms.restype = _dbl
    lib.pd_last_kernel_ms.argtypes = []
    lib.pd_device_status.restype = ci
    lib.pd_device_status.argtypes = [ctypes.POINTER(ci), ci, cp, sz]
    lib.pd_gray_scott_static.restype = ci
    lib.pd_gray_scott_static.argtypes = [ctypes.POINTER(GrayScottParams), ci, vp, vp, vp, vp, vp, cp, sz]
    lib.pd_gray_scott_slab_push.restype = ci
    lib.pd_gray_scott_slab_push.argtypes = [ctypes.POINTER(GrayScottParams), ci, vp, vp, vp, vp,
                                            ctypes.POINTER(GsNeighbours), vp, sz, vp, cp, sz]
    lib.pd_peer_alloc.restype = ci
    lib.pd_peer_alloc.argtypes = [sz, vpp, cp, sz]
    lib.pd_peer_export.restype = ci
    lib.pd_peer_export.argtypes = [vp, cp, cp, sz]
    lib.pd_peer_open.restype = ci
    lib.pd_peer_open.argtypes = [cp, vpp, cp, sz]
    lib.pd_peer_close.restype = ci
    lib.pd_peer_close.argtypes = [vp, cp, sz]
    lib.pd_peer_free.restype = ci
    lib.pd_peer_free.argtypes = [vp, cp, sz]
    lib.pd_custom_ode_check.restype = ci
    lib.pd_custom_ode_check.argtypes = [ctypes.POINTER(CustomOdeParams), sz, ci, cp, sz, cp, sz]
    lib.pd_custom_ode_source.restype = ci
    lib.pd_custom_ode_source.argtypes = [ctypes.POINTER(CustomOdeParams), sz, ci, cp, sz, szp, cp, sz]
    lib.pd_source_kernel_check.restype = ci
    lib.pd_source_kernel_check.argtypes = [ctypes.POINTER(SourceKernelParams), sz, ci, cp, sz, cp, sz]


def library() -> ctypes.CDLL:
    """Load the native library once per process (locked: concurrent first
    calls must not both run the body, as in src/palladium/ffi.py:64-79)."""
    global _lib
    if _lib is not None:
        return _lib
    with _LOAD_LOCK:
        if _lib is not None:
            return _lib
        path = library_path()
        if not path.is_file():
            raise EmitError(
                f"palladium_b200's CUDA library ({path}) isn't built. Build it with "
                "`python -m palladium_b200.build` (needs nvcc), or set PALLADIUM_FFI_LIBRARY "
                "to an existing build. There is no CPU fallback."
            )
        lib = ctypes.CDLL(str(path))
        _declare(lib)
        version = lib.pd_version()
        if version != PD_ABI_VERSION:
            raise EmitError(f"{path} has ABI version {version}, this package expects {PD_ABI_VERSION}; rebuild it")
        _lib = lib
    return _lib


_ERR_CAP = 4096


def _raise(code: int, message: bytes) -> None:
    text = message.decode("utf-8", "replace") or f"native call failed with status {code}"
    if code == 1:
        if "does not compile" in text:
            raise EmitError(text)
        raise DispatchError(text)
    if code == 3:
        raise DispatchError(text) if "no CUDA device" in text else PalladiumError(text)
    raise PalladiumError(text)


def _arrays(grid, block):
    """The grid and threadgroup as int64[3] arrays; cached, a call shape repeats (read-only use)."""
    try:
        return _arrays_cached(tuple(grid), block if block is None or isinstance(block, int) else tuple(block))
    except TypeError:       # unhashable or unusual sequence types take the plain route
        return _arrays_plain(grid, block)


@functools.lru_cache(maxsize=256)
def _arrays_cached(grid, block):
    return _arrays_plain(grid, block)


def _arrays_plain(grid, block):
    g = tuple(int(x) for x in grid) + (1, 1, 1)
    garr = (_i64 * 3)(*g[:3])
    if block is None:
        barr = (_i64 * 3)(0, 0, 0)
    else:
        b = (int(block),) if isinstance(block, int) else tuple(int(x) for x in block)
        b = b + (1, 1, 1)
        barr = (_i64 * 3)(*b[:3])
    return garr, barr


def _buffers(ptrs_and_bytes):
    n = len(ptrs_and_bytes)
    ptrs = (ctypes.c_void_p * max(n, 1))(*[p for p, _ in ptrs_and_bytes])
    sizes = (ctypes.c_size_t * max(n, 1))(*[b for _, b in ptrs_and_bytes])
    return n, ptrs, sizes


_thread_state = threading.local()


def _err_buffer():
    """One message buffer per thread (the native calls write it only on failure, NUL-terminated)."""
    buf = getattr(_thread_state, "err", None)
    if buf is None:
        buf = _thread_state.err = ctypes.create_string_buffer(_ERR_CAP)
    return buf


def launch(family: int, params: ctypes.Structure, math_mode: int, grid, block, inputs, outputs, stream: int = 0,
           workspace: tuple[int, int] | None = None) -> None:
    """pd_launch on device pointers. inputs / outputs: lists of (pointer, bytes)."""
    lib = library()
    garr, barr = _arrays(grid, block)
    n_in, in_ptrs, in_sizes = _buffers(inputs)
    n_out, out_ptrs, out_sizes = _buffers(outputs)
    err = _err_buffer()
    ws_ptr, ws_bytes = workspace if workspace else (None, 0)
    rc = lib.pd_launch(family, ctypes.addressof(params), ctypes.sizeof(params), math_mode, garr, barr, n_in, in_ptrs,
                       in_sizes, n_out, out_ptrs, out_sizes, ws_ptr, ws_bytes, stream or None, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)


def dispatch_host(family: int, params: ctypes.Structure, math_mode: int, grid, block, inputs, outputs) -> None:
    """pd_dispatch_host on host pointers (blocking)."""
    lib = library()
    garr, barr = _arrays(grid, block)
    n_in, in_ptrs, in_sizes = _buffers(inputs)
    n_out, out_ptrs, out_sizes = _buffers(outputs)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = lib.pd_dispatch_host(family, ctypes.addressof(params), ctypes.sizeof(params), math_mode, garr, barr, n_in,
                              in_ptrs, in_sizes, n_out, out_ptrs, out_sizes, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)


def submit_host(family: int, params: ctypes.Structure, math_mode: int, grid, block, inputs, out_sizes,
                out_ptrs=None, inputs_on_device: bool = False) -> int:
    """pd_submit_host: queue a call on host pointers without waiting for it; returns the ticket.
    inputs: (pointer, bytes) pairs, copied before the call returns; out_sizes: bytes per output;
    out_ptrs: page-locked result arrays to download into directly (else the results are collected
    by wait_host); inputs_on_device: the input pointers are device memory (uploaded earlier)."""
    lib = library()
    garr, barr = _arrays(grid, block)
    n_in, in_ptrs, in_sizes = _buffers(inputs)
    n_out = len(out_sizes)
    sizes = (ctypes.c_size_t * max(n_out, 1))(*out_sizes)
    outs = (ctypes.c_void_p * max(n_out, 1))(*out_ptrs) if out_ptrs is not None else None
    ticket = ctypes.c_uint64(0)
    err = _err_buffer()
    on_device = (ctypes.c_int * max(n_in, 1))(*([1] * n_in)) if inputs_on_device else None
    rc = lib.pd_submit_host(family, ctypes.addressof(params), ctypes.sizeof(params), math_mode, garr, barr, n_in,
                            in_ptrs, in_sizes, on_device, n_out, outs, sizes, ctypes.byref(ticket), err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return ticket.value


def wait_host(ticket: int, outputs) -> None:
    """pd_wait_host: block until the call behind `ticket` has finished and copy its results into
    `outputs` ((pointer, bytes) pairs; an empty list only retires the ticket)."""
    n_out, out_ptrs, out_sizes = _buffers(outputs)
    err = _err_buffer()
    rc = library().pd_wait_host(ctypes.c_uint64(ticket), n_out, out_ptrs, out_sizes, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)


def explain(family: int, params: ctypes.Structure, math_mode: int, grid, block) -> LaunchInfo:
    lib = library()
    garr, barr = _arrays(grid, block)
    info = LaunchInfo()
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = lib.pd_explain(family, ctypes.addressof(params), ctypes.sizeof(params), math_mode, garr, barr,
                        ctypes.byref(info), err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return info


def set_tuning(key: str, value: int) -> None:
    if library().pd_set_tuning(key.encode(), int(value)):
        raise KeyError(f"unknown tuning key {key!r}")


def get_tuning(key: str) -> int:
    out = _i64(0)
    if library().pd_get_tuning(key.encode(), ctypes.byref(out)):
        raise KeyError(f"unknown tuning key {key!r}")
    return int(out.value)


class thread_tuning:
    """Context manager: tuning knobs overridden for the calling thread only
    (pd_set_thread_tuning), restored on exit.  `with thread_tuning(gs_variant=1): call(...)`
    picks a kernel variant for that call without touching other threads' calls."""

    def __init__(self, **knobs: int):
        self.knobs = knobs

    def __enter__(self):
        lib = library()
        for key, value in self.knobs.items():
            if lib.pd_set_thread_tuning(key.encode(), int(value)):
                self.__exit__()
                raise KeyError(f"unknown tuning key {key!r}")
        return self

    def __exit__(self, *exc):
        lib = library()
        for key in self.knobs:
            lib.pd_clear_thread_tuning(key.encode())
        return False


def device_count() -> int:
    return int(library().pd_device_count())


def measure_fp32_fma_peak() -> float:
    out = _dbl(0.0)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_measure_fp32_fma_peak(ctypes.byref(out), err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return float(out.value)


def measure_int32_alu_peak() -> float:
    out = _dbl(0.0)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_measure_int32_alu_peak(ctypes.byref(out), err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return float(out.value)


def last_kernel_ms() -> float:
    return float(library().pd_last_kernel_ms())


def device_status(clear: bool = True) -> int:
    """pd_device_status: the code a kernel recorded on the current device when one of
    its bounded waits ran out (0: none).  Read it after synchronising the stream."""
    code = ctypes.c_int(0)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_device_status(ctypes.byref(code), 1 if clear else 0, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return int(code.value)


def gray_scott_static(params: GrayScottParams, math_mode: int, u: int, v: int, uo: int, vo: int,
                      stream: int = 0) -> None:
    """pd_gray_scott_static on device pointers: the multi-step stencil with its
    ping-pong fields in the library's fixed 8 MiB array instead of allocated
    scratch (at most 2^20 cells per call; calls on one device must not overlap)."""
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_gray_scott_static(ctypes.byref(params), math_mode, u, v, uo, vo, stream or None, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)


def custom_ode_check(params: CustomOdeParams, math_mode: int = 0) -> str:
    """pd_custom_ode_check: compile a run-time right-hand side for sm_100a without
    a device; returns the compiler's log (warnings), raises EmitError on errors."""
    log = ctypes.create_string_buffer(_ERR_CAP)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_custom_ode_check(ctypes.byref(params), ctypes.sizeof(params), math_mode, log, _ERR_CAP, err,
                                       _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return log.value.decode("utf-8", "replace")


def source_kernel_check(params: SourceKernelParams, math_mode: int = 0) -> str:
    """pd_source_kernel_check: the same for a complete caller-written kernel."""
    log = ctypes.create_string_buffer(_ERR_CAP)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_source_kernel_check(ctypes.byref(params), ctypes.sizeof(params), math_mode, log, _ERR_CAP, err,
                                          _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return log.value.decode("utf-8", "replace")


def custom_ode_source(params: CustomOdeParams, math_mode: int = 2) -> str:
    """pd_custom_ode_source: the generated CUDA text of a run-time right-hand side call."""
    err = ctypes.create_string_buffer(_ERR_CAP)
    needed = ctypes.c_size_t(0)
    lib = library()
    rc = lib.pd_custom_ode_source(ctypes.byref(params), ctypes.sizeof(params), math_mode, None, 0,
                                  ctypes.byref(needed), err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    out = ctypes.create_string_buffer(needed.value)
    rc = lib.pd_custom_ode_source(ctypes.byref(params), ctypes.sizeof(params), math_mode, out, needed.value, None,
                                  err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return out.value.decode("utf-8", "replace")


def gray_scott_slab_push(params: GrayScottParams, math_mode: int, u: int, v: int, uo: int, vo: int,
                         neighbours: GsNeighbours, stream: int = 0) -> None:
    """pd_gray_scott_slab_push on device pointers: a slab call whose final launch
    also stores the boundary rows into the neighbours' ghost rows (peer memory)."""
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_gray_scott_slab_push(ctypes.byref(params), math_mode, u, v, uo, vo, ctypes.byref(neighbours),
                                           None, 0, stream or None, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)


def peer_alloc(nbytes: int) -> int:
    out = ctypes.c_void_p()
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_peer_alloc(int(nbytes), ctypes.byref(out), err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return int(out.value)


def peer_export(ptr: int) -> bytes:
    handle = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_peer_export(ptr, handle, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return handle.raw


def peer_open(handle: bytes) -> int:
    out = ctypes.c_void_p()
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_peer_open(ctypes.create_string_buffer(handle, PEER_HANDLE_BYTES), ctypes.byref(out), err,
                                _ERR_CAP)
    if rc:
        _raise(rc, err.value)
    return int(out.value)


def peer_close(ptr: int) -> None:
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_peer_close(ptr, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)


def peer_free(ptr: int) -> None:
    err = ctypes.create_string_buffer(_ERR_CAP)
    rc = library().pd_peer_free(ptr, err, _ERR_CAP)
    if rc:
        _raise(rc, err.value)
