"""jax.ffi registration of the CUDA handler (used only when JAX is installed).

Mirrors `_register` / `FfiCallable.__call__` of the reference
(src/palladium/ffi.py:64-79,163-187): the shim `csrc/pd_xla_ffi.cc` is compiled
against `jax.ffi.include_dir()` on first use, loaded with ctypes, registered
once per process under a lock, and called with the family id, the parameter
block, grid, threadgroup and math_mode as attributes.

JAX is not present where this package is built and tested, so this module is
exercised only by import; `cuda_call_jit` reaches it only when handed JAX values.
"""

from __future__ import annotations

import ctypes
import subprocess
import threading
from pathlib import Path

import numpy as np

from . import _native
from .errors import EmitError

_TARGET_NAME = "palladium_cuda_dispatch"
_SOURCE_TARGET_NAME = "palladium_cuda_dispatch_source"
_PKG = Path(__file__).resolve().parent
_SHIM = _PKG / "libpalladium_xla_ffi.so"
_REGISTER_LOCK = threading.Lock()
_registered = False


def build_shim() -> Path:
    """Compile csrc/pd_xla_ffi.cc against JAX's FFI headers and link it to the CUDA library."""
    import jax

    include = jax.ffi.include_dir()
    src = _PKG / "csrc" / "pd_xla_ffi.cc"
    lib = _native.library_path()
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-I{include}", str(src), "-o", str(_SHIM),
           f"-L{lib.parent}", f"-l:{lib.name}", f"-Wl,-rpath,{lib.parent}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise EmitError(f"building the XLA-FFI shim failed:\n{proc.stderr}")
    return _SHIM


def _register() -> None:
    global _registered
    if _registered:
        return
    with _REGISTER_LOCK:
        if _registered:
            return
        import jax

        if not _SHIM.is_file():
            build_shim()
        _native.library()
        handle = ctypes.CDLL(str(_SHIM))
        jax.ffi.register_ffi_target(_TARGET_NAME, jax.ffi.pycapsule(handle.palladium_cuda_dispatch), platform="cpu")
        jax.ffi.register_ffi_target(_SOURCE_TARGET_NAME, jax.ffi.pycapsule(handle.palladium_cuda_dispatch_source),
                                    platform="cpu")
        _registered = True


def ffi_call(callable_, args):
    """Dispatch `callable_` (an FfiCallable) on JAX values via jax.ffi."""
    import jax

    _register()
    shapes = tuple((tuple(a.shape), np.dtype(a.dtype).name) for a in args)
    spec, _ = callable_._entry(shapes)
    grid = tuple(spec.grid) + (1, 1, 1)
    tg = callable_._threadgroup
    tg = (0, 0, 0) if tg is None else (((tg,) if isinstance(tg, int) else tuple(tg)) + (1, 1))[:3]
    out_structs = [jax.ShapeDtypeStruct(info.array_shape, info.dtype) for info in spec.outputs]
    result_shapes = out_structs[0] if len(out_structs) == 1 else out_structs
    params = np.frombuffer(bytes(spec.params), dtype=np.uint8)
    target, text = _TARGET_NAME, {}
    constants = spec.family.constants
    if spec.family.name == "source":
        # source text travels as string attributes, as msl_source / function_name do in the reference
        target = _SOURCE_TARGET_NAME
        text = dict(cuda_source=constants["source"], function_name=constants["function_name"])
    elif spec.family.name == "custom_ode":
        target = _SOURCE_TARGET_NAME
        text = dict(cuda_source=constants["rhs"], function_name="")
    return jax.ffi.ffi_call(target, result_shapes, vmap_method=callable_._vmap_method)(
        *args, **text, family=np.int64(spec.family.family_id), params=params, grid_x=np.int64(grid[0]),
        grid_y=np.int64(grid[1]), grid_z=np.int64(grid[2]), threadgroup_x=np.int64(tg[0]),
        threadgroup_y=np.int64(tg[1]), threadgroup_z=np.int64(tg[2]), math_mode=np.int64(callable_._math_mode))
