"""palladium_b200: the ensemble-integrator hot path of palladium on B200.

Pipeline of the reference: trace (Pallas -> KernelSpec) -> emit (KernelSpec ->
MSL) -> bind (MSL -> callable) behind `metal_call` (src/palladium/__init__.py:1-7).
Here: trace (validate a `pallas_call`-shaped request against a hand-written
kernel family) -> bind (family -> C-ABI launch in libpalladium_cuda.so) behind
`cuda_call`, which keeps `metal_call`'s signature, `.interpret`, `.explain`,
`.pin` and `.cache`; `cuda_call_jit` mirrors `metal_call_jit`.
"""

from __future__ import annotations

import threading
from collections.abc import Callable
from typing import Any

import numpy as np

from . import families, pl, workloads
from .diagnostics import KernelDiagnostics, explain_spec, log_compile
from .dispatch import BoundKernel, PendingResult, bind
from .errors import (
    DispatchError,
    EmitError,
    PalladiumError,
    TraceError,
    UnsupportedPrimitiveError,
)
from .families import BlockInfo, Family, KernelSpec, trace
from .ffi import FfiCallable, cuda_call_jit
from .interpret import interpret_callable, register_interpret_provider
from .math_mode import MathMode
from .stepping import Stepper

__all__ = [
    "BlockInfo",
    "BoundKernel",
    "CudaCallable",
    "DispatchError",
    "EmitError",
    "Family",
    "FfiCallable",
    "KernelDiagnostics",
    "KernelSpec",
    "MathMode",
    "PalladiumError",
    "PendingResult",
    "Stepper",
    "TraceError",
    "UnsupportedPrimitiveError",
    "bind",
    "cuda_call",
    "cuda_call_jit",
    "debug_msl",
    "families",
    "pl",
    "register_interpret_provider",
    "trace",
    "workloads",
]

__version__ = "0.1.0"

CacheKey = tuple[tuple[tuple[int, ...], str], ...]

# Element types the kernels take (the reference's table is emit.core.CTYPES).
_SUPPORTED_DTYPES = ("float32", "uint32", "int32")


def _check_dtypes(args: tuple) -> None:
    """Reject unsupported element types before tracing, with the fix in the
    message (src/palladium/__init__.py:58-80)."""
    for i, a in enumerate(args):
        dtype = getattr(a, "dtype", None)
        name = np.dtype(dtype if dtype is not None else np.asarray(a).dtype).name
        if name not in _SUPPORTED_DTYPES:
            hint = (
                "; float64 usually means jax_enable_x64 is on, disable it or cast to float32"
                if name == "float64"
                else ""
            )
            raise DispatchError(
                f"argument {i} has dtype {name}, which palladium cannot lower "
                f"(supported: {', '.join(_SUPPORTED_DTYPES)}){hint}"
            )


class CudaCallable:
    """A kernel family behind a `pl.pallas_call`-shaped call
    (the counterpart of MetalCallable, src/palladium/__init__.py:83-159).

    Attributes
    ----------
    interpret : callable
        The CPU oracle for the same call: the user's Pallas function under
        `pl.pallas_call(..., interpret=True)` when JAX is installed and the
        family carries one, else the registered interpret provider.
    cache : dict
        Input-shape signature -> `BoundKernel`.
    """

    def __init__(self, kernel: Family, pallas_kwargs: dict[str, Any], math_mode: Any,
                 threadgroup: int | tuple[int, ...] | None) -> None:
        if not isinstance(kernel, Family):
            raise UnsupportedPrimitiveError(
                "cuda_call needs a kernel family from palladium_b200.families (there is no "
                f"Pallas-to-CUDA emitter); got {type(kernel).__name__}"
            )
        self._family = kernel
        self._pallas_kwargs = dict(pallas_kwargs)
        self._math_mode = math_mode
        self._threadgroup = threadgroup
        # Validate the static part of the request now: a malformed grid or
        # out_shape should fail where the call is built, like a bad pallas_call.
        trace(kernel, self._pallas_kwargs)
        self.interpret = interpret_callable(kernel, self._pallas_kwargs)
        self.cache: dict[CacheKey, BoundKernel] = {}
        # Guards the cache-miss path: concurrent first calls on the same shape
        # must bind exactly once (src/palladium/__init__.py:112-114).
        self._lock = threading.Lock()

    def explain(self, *args) -> KernelDiagnostics:
        """Launch geometry for these inputs (arrays or ShapeDtypeStructs; no
        data is read, nothing is launched)."""
        _check_dtypes(args)
        return explain_spec(trace(self._family, self._pallas_kwargs, *args), self._threadgroup, self._math_mode)

    def pin(self, *args) -> Callable[[], np.ndarray | tuple[np.ndarray, ...]]:
        """Upload the inputs once; return a zero-argument callable that
        re-dispatches on the device-resident buffers."""
        arrays = [np.asarray(a) for a in args]
        self._bound(arrays)
        key: CacheKey = tuple((a.shape, a.dtype.str) for a in arrays)
        return self.cache[key].pinned(*arrays)

    def _bound(self, arrays: list[np.ndarray]) -> BoundKernel:
        key: CacheKey = tuple((a.shape, a.dtype.str) for a in arrays)
        bound = self.cache.get(key)
        if bound is None:
            with self._lock:
                bound = self.cache.get(key)
                if bound is None:
                    _check_dtypes(tuple(arrays))
                    spec = trace(self._family, self._pallas_kwargs, *arrays)
                    log_compile(spec, self._threadgroup, self._math_mode)
                    bound = bind(spec, math_mode=self._math_mode, threadgroup=self._threadgroup)
                    self.cache[key] = bound
        return bound

    def launch(self, *args) -> PendingResult:
        """Commit one dispatch without waiting (BoundKernel.launch)."""
        arrays = [np.asarray(a) for a in args]
        return self._bound(arrays).launch(*arrays)

    def __call__(self, *args) -> np.ndarray | tuple[np.ndarray, ...]:
        """Run the kernel on the GPU; NumPy in, NumPy out."""
        arrays = [np.asarray(a) for a in args]
        return self._bound(arrays)(*arrays)


def debug_msl(kernel: Family, *example_args, **pallas_kwargs) -> str:
    """The reference returns the emitted MSL for a call
    (src/palladium/__init__.py:162-190).  For the run-time compiled families
    the text returned is the CUDA source handed to the compiler (the generated
    integrator around a `custom_ode` right-hand side; a `source_kernel`'s own
    text).  The other kernels are precompiled, so for them it is the launch
    record: kernel name, constants, CUDA launch geometry and the source file
    the kernel is built from."""
    from . import _native
    from .math_mode import math_mode_ordinal

    math_mode = pallas_kwargs.pop("math_mode", MathMode.FAST)
    threadgroup = pallas_kwargs.pop("threadgroup", None)
    spec = trace(kernel, pallas_kwargs, *example_args)
    diag = explain_spec(spec, threadgroup, math_mode)
    if kernel.name == "custom_ode":
        return f"// {diag}\n" + _native.custom_ode_source(spec.params, math_mode_ordinal(math_mode))
    if kernel.name == "source":
        return f"// {diag}\n" + kernel.constants["source"]
    return (f"// {diag}\n// family: {kernel.name}\n// constants: {kernel.constants}\n"
            f"// source: palladium_b200/csrc/pd_kernels.cu\n")


def cuda_call(kernel: Family, **pallas_kwargs) -> CudaCallable:
    """`metal_call`, but the kernel runs on a B200 (src/palladium/__init__.py:193-226).

    Parameters
    ----------
    kernel : Family
        A kernel family from `palladium_b200.families`.
    **pallas_kwargs
        The usual `pl.pallas_call` keywords (out_shape, grid, in_specs,
        out_specs), plus `math_mode` (`MathMode`, FAST by default, as in the
        reference) and `threadgroup` (CUDA block size; None lets the library
        choose).

    Notes
    -----
    FAST reorders float arithmetic and uses approximate transcendentals; SAFE
    keeps IEEE operation order and matches the CPU oracle bit for bit where the
    arithmetic is IEEE-exact.
    """
    math_mode = pallas_kwargs.pop("math_mode", MathMode.FAST)
    threadgroup = pallas_kwargs.pop("threadgroup", None)
    return CudaCallable(kernel, pallas_kwargs, math_mode, threadgroup)
