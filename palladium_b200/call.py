"""`cuda_call`: a kernel family behind a `pl.pallas_call`-shaped call, NumPy in
and NumPy out.

The counterpart of the reference's `metal_call` / `MetalCallable`
(src/palladium/__init__.py:83-159,193-226).  What a user sees is the same --
build the call once from `grid / in_specs / out_specs / out_shape` plus
`math_mode` and `threadgroup`, then call it with arrays; `.interpret` is the CPU
oracle for the same call, `.explain(*args)` reports the launch without running
it, `.pin(*arrays)` keeps inputs on the device, `.cache` holds one bound kernel
per input signature.  Underneath, a call validates its description against the
family (`families.trace`), binds it to the native library once per signature
and from then on only moves buffers.
"""

from __future__ import annotations

import threading
from collections.abc import Callable, Hashable
from typing import Any

import numpy as np

from .diagnostics import KernelDiagnostics, explain_spec, log_compile
from .dispatch import BoundKernel, PendingResult, bind
from .errors import DispatchError, UnsupportedPrimitiveError
from .families import Family, trace
from .interpret import interpret_callable
from .math_mode import MathMode, math_mode_ordinal

# Element types the kernels take (the reference's table is emit.core.CTYPES).
SUPPORTED_DTYPES = ("float32", "uint32", "int32")

Signature = tuple[tuple[tuple[int, ...], str], ...]


def require_supported_dtypes(operands) -> None:
    """Refuse element types no kernel takes, before anything is traced, and say
    what to do about the usual culprit (the wording users of the reference know,
    src/palladium/__init__.py:58-80)."""
    names = []
    for operand in operands:
        dtype = getattr(operand, "dtype", None)
        names.append(np.dtype(np.asarray(operand).dtype if dtype is None else dtype).name)
    for position, name in enumerate(names):
        if name in SUPPORTED_DTYPES:
            continue
        advice = ""
        if name == "float64":
            advice = "; float64 usually means jax_enable_x64 is on, disable it or cast to float32"
        raise DispatchError(f"argument {position} has dtype {name}, which palladium cannot lower "
                            f"(supported: {', '.join(SUPPORTED_DTYPES)}){advice}")


def signature_of(arrays) -> Signature:
    return tuple((a.shape, a.dtype.str) for a in arrays)


class _BindOnce(dict):
    """signature -> BoundKernel, filled by at most one thread per signature:
    sixteen threads making the first call on one shape must bind once
    (the reference tests exactly that, tests/test_17_robustness.py:22-51)."""

    def __init__(self) -> None:
        super().__init__()
        self._guard = threading.Lock()

    def obtain(self, key: Hashable, make: Callable[[], BoundKernel]) -> BoundKernel:
        found = self.get(key)
        if found is not None:
            return found
        with self._guard:
            found = self.get(key)          # somebody else may have bound it meanwhile
            if found is None:
                found = self[key] = make()
        return found


class CudaCallable:
    """What `cuda_call` returns.

    Attributes
    ----------
    interpret : callable
        The CPU oracle for the same call: the user's Pallas function under
        `pl.pallas_call(..., interpret=True)` when JAX is installed and the
        family carries one, else the registered interpret provider.
    cache : dict
        Input signature ((shape, dtype string) per array) -> `BoundKernel`.
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
        trace(kernel, self._pallas_kwargs)      # a malformed grid / out_shape fails here, where the call is built
        self.interpret = interpret_callable(kernel, self._pallas_kwargs)
        self.cache: dict[Signature, BoundKernel] = _BindOnce()

    # -- binding ----------------------------------------------------------------------
    def _bind_for(self, arrays: list[np.ndarray]) -> BoundKernel:
        require_supported_dtypes(arrays)
        spec = trace(self._family, self._pallas_kwargs, *arrays)
        log_compile(spec, self._threadgroup, self._math_mode)
        return bind(spec, math_mode=self._math_mode, threadgroup=self._threadgroup)

    def _bound(self, arrays: list[np.ndarray]) -> BoundKernel:
        return self.cache.obtain(signature_of(arrays), lambda: self._bind_for(arrays))

    # -- the four ways to use it ---------------------------------------------------------
    def __call__(self, *args) -> np.ndarray | tuple[np.ndarray, ...]:
        """Upload, run on the GPU, download."""
        arrays = [np.asarray(a) for a in args]
        return self._bound(arrays)(*arrays)

    def launch(self, *args) -> PendingResult:
        """Enqueue one dispatch and return at once; `.wait()` on the result downloads."""
        arrays = [np.asarray(a) for a in args]
        return self._bound(arrays).launch(*arrays)

    def pin(self, *args) -> Callable[[], np.ndarray | tuple[np.ndarray, ...]]:
        """Upload the inputs once and return a zero-argument callable that
        re-dispatches on the device-resident copies (later changes to the
        arrays passed here are not seen)."""
        arrays = [np.asarray(a) for a in args]
        return self._bound(arrays).pinned(*arrays)

    def explain(self, *args) -> KernelDiagnostics:
        """The launch these inputs would get.  `args` may be arrays or
        ShapeDtypeStructs; no data is read and nothing is launched."""
        require_supported_dtypes(args)
        return explain_spec(trace(self._family, self._pallas_kwargs, *args), self._threadgroup, self._math_mode)


def cuda_call(kernel: Family, **pallas_kwargs) -> CudaCallable:
    """Build a GPU call from a kernel family and the keywords of `pl.pallas_call`.

    kernel: one of `palladium_b200.families` (with its constants).
    grid, in_specs, out_specs, out_shape: as for `pl.pallas_call`; they are
    checked against what the family launches.
    math_mode: `MathMode` or its name; FAST unless said otherwise, as in the
    reference.  FAST reorders float arithmetic and uses approximate
    transcendentals; SAFE keeps IEEE operation order and equals the CPU oracle bit
    for bit where the arithmetic is IEEE-exact (use it for compensated arithmetic).
    threadgroup: CUDA block size; None leaves the choice to the library."""
    options = dict(pallas_kwargs)
    math_mode = options.pop("math_mode", MathMode.FAST)
    threadgroup = options.pop("threadgroup", None)
    return CudaCallable(kernel, options, math_mode, threadgroup)


def debug_msl(kernel: Family, *example_args, **pallas_kwargs) -> str:
    """Text describing what a call would run (the reference returns the emitted
    MSL, src/palladium/__init__.py:162-190).  For the run-time compiled families
    this is the CUDA source handed to the compiler: the generated integrator
    around a `custom_ode` right-hand side, or a `source_kernel`'s own text.  The
    other kernels are precompiled; for them it is the launch record (kernel name,
    constants, CUDA launch geometry, the file the kernel is built from)."""
    from . import _native

    options = dict(pallas_kwargs)
    math_mode = options.pop("math_mode", MathMode.FAST)
    threadgroup = options.pop("threadgroup", None)
    spec = trace(kernel, options, *example_args)
    header = f"// {explain_spec(spec, threadgroup, math_mode)}\n"
    if kernel.name == "custom_ode":
        return header + _native.custom_ode_source(spec.params, math_mode_ordinal(math_mode))
    if kernel.name == "source":
        return header + kernel.constants["source"]
    return (header + f"// family: {kernel.name}\n// constants: {kernel.constants}\n"
            "// source: palladium_b200/csrc/pd_kernels.cu\n")
