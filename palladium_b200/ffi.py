"""`cuda_call_jit`: the kernel as one node of a larger device-side program.

The reference's `metal_call_jit` registers its native handler as an XLA FFI
target so a kernel call composes inside `jax.jit` next to `jnp` ops
(src/palladium/ffi.py:90-221).  The same C entry points serve three callers
here, chosen by the argument type:

* torch CUDA tensors: `pd_launch` on the current torch stream, no host
  synchronisation, tensors out -- the call is stream-ordered with the torch
  ops around it and can be captured in a CUDA graph with them;
* NumPy arrays (host buffers, what an XLA:CPU handler receives):
  `pd_dispatch_host`, which uploads, launches, downloads and blocks, the
  contract of the reference handler (native/ffi/palladium_ffi.cpp:150-188);
* JAX arrays / tracers, when JAX and the XLA-FFI shim are present:
  `jax.ffi.ffi_call` with the family id, constants, grid, threadgroup and
  math_mode as attributes (csrc/pd_xla_ffi.cc).

`vmap_method` is validated exactly as the reference does
(src/palladium/ffi.py:87,118-125).
"""

from __future__ import annotations

import importlib.util
import threading
from typing import Any

import numpy as np

from . import _native
from .diagnostics import KernelDiagnostics, explain_spec, log_compile
from .dispatch import BoundKernel, bind
from .errors import DispatchError, UnsupportedPrimitiveError
from .families import Family, KernelSpec, trace
from .interpret import interpret_callable
from .math_mode import MathMode, math_mode_ordinal
from .pl import ShapeDtypeStruct

__all__ = ["FfiCallable", "cuda_call_jit"]

_TARGET_NAME = "palladium_cuda_dispatch"

# ffi_call batching methods that re-invoke the target once per batch element:
# the launch grid is fixed per unbatched shape, so whole-batch methods would
# run it over batched buffers (src/palladium/ffi.py:82-87).
_SAFE_VMAP_METHODS = (None, "sequential", "sequential_unrolled")


def _is_torch_tensor(x) -> bool:
    mod = type(x).__module__
    return mod.startswith("torch") and hasattr(x, "data_ptr")


def _is_jax_value(x) -> bool:
    return type(x).__module__.startswith(("jax", "jaxlib"))


_DTYPE_TABLES: list = []
_SMALL_HOST_CALL_BYTES = 256 << 10


def _torch_dtype_tables(torch):
    """(torch dtype -> NumPy dtype name, and back), built once."""
    if not _DTYPE_TABLES:
        to_np = {torch.float32: "float32", torch.int32: "int32", torch.uint32: "uint32", torch.float64: "float64",
                 torch.uint8: "uint8"}
        to_torch = {"float32": torch.float32, "int32": torch.int32, "uint32": torch.uint32, "float64": torch.float64}
        _DTYPE_TABLES.append((to_np, to_torch))
    return _DTYPE_TABLES[0]


def _pinned_empty(shape, dtype) -> np.ndarray:
    """Output array in page-locked host memory (torch's caching host allocator),
    so the device-to-host copy is a true asynchronous DMA and the chunks of a
    pipelined call overlap; falls back to ordinary memory without CUDA."""
    try:
        import torch

        if torch.cuda.is_available():
            nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
            buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, pin_memory=True)
            return buf.numpy()[:nbytes].view(dtype).reshape(shape)
    except Exception:
        pass
    return np.empty(shape, dtype)


class FfiCallable:
    """A kernel family callable on device tensors (stream-ordered), host
    arrays (blocking), or JAX values (through jax.ffi when available).

    Attributes
    ----------
    interpret : callable
        The CPU oracle for the same call (see `CudaCallable.interpret`).
    """

    def __init__(self, kernel: Family, pallas_kwargs: dict[str, Any], math_mode: Any,
                 vmap_method: str | None = None, threadgroup=None) -> None:
        if vmap_method not in _SAFE_VMAP_METHODS:
            raise ValueError(
                f"vmap_method {vmap_method!r} is not supported: the launch "
                "grid is baked per unbatched shape, so whole-batch methods "
                "would dispatch it over batched buffers. Use 'sequential' "
                "or 'sequential_unrolled' (one dispatch per batch element), "
                "or put the batch dimension in the Pallas grid instead."
            )
        if not isinstance(kernel, Family):
            raise UnsupportedPrimitiveError(
                "cuda_call_jit needs a kernel family from palladium_b200.families; "
                f"got {type(kernel).__name__}"
            )
        self._family = kernel
        self._pallas_kwargs = dict(pallas_kwargs)
        self._math_mode = math_mode_ordinal(math_mode)
        self._vmap_method = vmap_method
        self._threadgroup = threadgroup
        trace(kernel, self._pallas_kwargs)
        self.interpret = interpret_callable(kernel, self._pallas_kwargs)
        self._cache: dict[tuple, tuple[KernelSpec, BoundKernel]] = {}
        self._lock = threading.Lock()

    def explain(self, *args) -> KernelDiagnostics:
        return explain_spec(trace(self._family, self._pallas_kwargs, *args), self._threadgroup, self._math_mode)

    def _entry(self, shapes: tuple) -> tuple[KernelSpec, BoundKernel]:
        entry = self._cache.get(shapes)
        if entry is None:
            with self._lock:
                entry = self._cache.get(shapes)
                if entry is None:
                    structs = [ShapeDtypeStruct(s, np.dtype(d)) for s, d in shapes]
                    spec = trace(self._family, self._pallas_kwargs, *structs)
                    log_compile(spec, self._threadgroup, self._math_mode)
                    entry = (spec, bind(spec, math_mode=self._math_mode, threadgroup=self._threadgroup))
                    self._cache[shapes] = entry
        return entry

    def __call__(self, *args):
        if args and all(_is_torch_tensor(a) for a in args):
            return self._call_torch(args)
        if args and any(_is_jax_value(a) for a in args):
            return self._call_jax(args)
        return self._call_host(args)

    def vmap(self, *args, in_axes=0):
        """The call mapped over a leading batch axis, one dispatch per batch
        element: what `jax.vmap` does to the reference's FFI call under
        `vmap_method="sequential"` (src/palladium/ffi.py:118-125, 190-221).  As
        there, a call built without a `vmap_method` refuses to be batched.
        `in_axes`: 0 (every operand carries the batch axis first) or a sequence
        with 0 / None per operand (None: the operand is shared by all elements).
        Outputs are stacked along a new leading axis."""
        if self._vmap_method is None:
            raise NotImplementedError(
                "this call was built without vmap_method: batching it needs "
                "vmap_method='sequential' (or 'sequential_unrolled'), one dispatch per batch element")
        axes = [in_axes] * len(args) if in_axes in (0, None) else list(in_axes)
        if len(axes) != len(args) or any(a not in (0, None) for a in axes):
            raise ValueError("in_axes must be 0, None, or one of them per operand")
        sizes = {int(a.shape[0]) for a, ax in zip(args, axes) if ax == 0}
        if len(sizes) != 1:
            raise ValueError(f"mapped operands disagree on the batch size: {sorted(sizes)}")
        batch = sizes.pop()
        results = [self(*[a[i] if ax == 0 else a for a, ax in zip(args, axes)]) for i in range(batch)]
        single = not isinstance(results[0], (tuple, list))
        columns = [[r] for r in results] if single else [list(r) for r in results]
        stacked = []
        for k in range(len(columns[0])):
            parts = [row[k] for row in columns]
            if _is_torch_tensor(parts[0]):
                import torch

                stacked.append(torch.stack(parts))
            else:
                stacked.append(np.stack(parts))
        return stacked[0] if single else tuple(stacked)

    # ---- torch CUDA tensors: stream-ordered, no synchronisation ----------------
    def _call_torch(self, args, out=None):
        import torch

        np_dtype, torch_dtype = _torch_dtype_tables(torch)
        shapes = tuple((tuple(a.shape), np_dtype.get(a.dtype, str(a.dtype))) for a in args)
        spec, bound = self._entry(shapes)
        device = args[0].device if args else torch.device("cuda", torch.cuda.current_device())
        if out is not None:
            outs = list(out) if isinstance(out, (list, tuple)) else [out]
        else:
            outs = [torch.empty(info.array_shape, dtype=torch_dtype[info.dtype.name], device=device)
                    for info in spec.outputs]
        bound.launch_device(list(args), outs)
        return outs[0] if len(outs) == 1 else tuple(outs)

    def on_device(self, *args, out=None):
        """Stream-ordered launch returning torch CUDA tensors, also for families
        without inputs (where `__call__` cannot tell a device call from a host call).
        `out`: preallocated contiguous output tensors (views are fine) to write into."""
        return self._call_torch(args, out)

    # ---- host buffers: the XLA:CPU handler contract -----------------------------
    def _call_host(self, args):
        arrays = [np.ascontiguousarray(a) for a in args]
        shapes = tuple((a.shape, a.dtype.name) for a in arrays)
        spec, _ = self._entry(shapes)
        out_bytes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.outputs]
        if sum(a.nbytes for a in arrays) + sum(out_bytes) < _SMALL_HOST_CALL_BYTES:
            # A small call: inputs packed into one upload, results into one download (the library's
            # slot path), ordinary result arrays -- cheaper than page-locked ones at this size.
            outs = [np.empty(info.array_shape, info.dtype) for info in spec.outputs]
            ticket = _native.submit_host(spec.family.family_id, spec.params, self._math_mode, spec.grid,
                                         self._threadgroup, [(a.ctypes.data, a.nbytes) for a in arrays], out_bytes)
            _native.wait_host(ticket, [(o.ctypes.data, o.nbytes) for o in outs])
            return outs[0] if len(outs) == 1 else tuple(outs)
        outs = [_pinned_empty(info.array_shape, info.dtype) for info in spec.outputs]
        _native.dispatch_host(
            spec.family.family_id, spec.params, self._math_mode, spec.grid, self._threadgroup,
            [(a.ctypes.data, a.nbytes) for a in arrays],
            [(o.ctypes.data, o.nbytes) for o in outs],
        )
        return outs[0] if len(outs) == 1 else tuple(outs)

    # ---- JAX values: jax.ffi, when JAX and the compiled shim exist --------------
    def _call_jax(self, args):
        if importlib.util.find_spec("jax") is None:
            raise DispatchError("JAX values were passed but JAX is not installed")
        from . import xla_ffi

        return xla_ffi.ffi_call(self, args)


def cuda_call_jit(kernel: Family, **pallas_kwargs) -> FfiCallable:
    """`metal_call_jit` for B200 (src/palladium/ffi.py:190-221): the usual
    `pl.pallas_call` keywords plus `math_mode` (FAST by default), `threadgroup`
    and `vmap_method` ('sequential' / 'sequential_unrolled'; None, the default,
    rejects `jax.vmap`)."""
    math_mode = pallas_kwargs.pop("math_mode", MathMode.FAST)
    vmap_method = pallas_kwargs.pop("vmap_method", None)
    threadgroup = pallas_kwargs.pop("threadgroup", None)
    return FfiCallable(kernel, pallas_kwargs, math_mode, vmap_method, threadgroup)
