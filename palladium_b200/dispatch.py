"""Bind a validated call to the native library and run it.

The reference's step 3 (src/palladium/dispatch.py:90-314): `bind(spec, ...)`
returns a `BoundKernel` whose `launch(*arrays)` commits one dispatch without
blocking and returns a `PendingResult`; `__call__` is `launch(...).wait()`;
`pinned(*arrays)` uploads once and returns a zero-argument re-dispatcher.
Argument count, dtype and shape are checked strictly and never cast
(src/palladium/dispatch.py:150-176).

Device memory, pinned staging buffers, streams and events come from PyTorch;
the kernels are launched through the C ABI (`pd_launch`) on the kernel's own
stream.  All buffers are handled as raw bytes, so no dtype conversion can
happen on the way.  There is no CPU path: without a CUDA device `launch`
raises DispatchError.
"""

from __future__ import annotations

import dataclasses
import os
import threading
from collections.abc import Callable
from pathlib import Path

import numpy as np

from . import _native
from .errors import DispatchError, PalladiumError
from .families import KernelSpec
from .math_mode import MathMode, math_mode_ordinal

__all__ = ["BoundKernel", "PendingResult", "bind"]

_DIRECT_OUTPUT_BYTES = 256 << 10   # results at least this large download into page-locked arrays of their own


def _torch():
    import torch

    return torch


def _require_cuda():
    torch = _torch()
    if not torch.cuda.is_available():
        raise DispatchError(
            "no CUDA device is available: palladium_b200 kernels run on the GPU only "
            "(there is no CPU fallback; use `.interpret` for a CPU oracle)"
        )
    return torch


def _dump_source(spec: KernelSpec, math_mode) -> None:
    """PALLADIUM_DUMP_MSL=1 prints, and a directory path writes, a record of the
    kernel being bound (the reference dumps the MSL text,
    src/palladium/dispatch.py:27-38; here the source is fixed, so the record
    names the CUDA source file, the family constants and the launch plan)."""
    dump = os.environ.get("PALLADIUM_DUMP_MSL")
    if not dump:
        return
    from .diagnostics import explain_spec

    src = Path(__file__).resolve().parent / "csrc" / "pd_kernels.cu"
    text = (f"// palladium kernel: {spec.name}\n// source: {src}\n// constants: {spec.family.constants}\n"
            f"// {explain_spec(spec, None, math_mode)}\n")
    if dump == "1" or dump.lower() == "stdout":
        print(text)
        return
    directory = Path(dump)
    directory.mkdir(parents=True, exist_ok=True)
    (directory / f"{spec.name}_{abs(hash(str(spec.family.constants))) % (1 << 48):012x}.txt").write_text(text)


class PendingResult:
    """A launched call whose kernels may still be executing.

    `wait()` blocks until the call has finished and returns the outputs as NumPy
    arrays (a bare array for one output), the contract of
    src/palladium/dispatch.py:66-86.  A second `wait()` returns the same arrays."""

    def __init__(self, out_infos: tuple, ticket: int, out_host: list | None = None) -> None:
        self.out_infos = out_infos
        self._ticket = ticket          # the library's handle of the call in flight (pd_submit_host)
        self.out_host = out_host       # page-locked arrays the results download into, or None (collected at the wait)
        self._result = None
        self._lock = threading.Lock()

    def _finish(self):
        ticket, self._ticket = self._ticket, None
        # A kernel whose bounded wait ran out recorded a code instead of computing: the native wait
        # reports it (PalladiumError) rather than hand over fields that were never written.
        if self.out_host is not None:
            _native.wait_host(ticket, [])
            return tuple(host.numpy()[: int(np.prod(info.array_shape)) * info.dtype.itemsize].view(info.dtype)
                         .reshape(info.array_shape) for host, info in zip(self.out_host, self.out_infos))
        outs = [np.empty(info.array_shape, info.dtype) for info in self.out_infos]
        _native.wait_host(ticket, [(o.ctypes.data, o.nbytes) for o in outs])
        return tuple(outs)

    def wait(self):
        with self._lock:
            if self._result is None:
                self._result = self._finish()
            outs = self._result
        return outs[0] if len(outs) == 1 else outs

    def __del__(self):
        # a result nobody waited for still holds a slot of the library: give it back
        ticket = getattr(self, "_ticket", None)
        if ticket is not None:
            try:
                _native.wait_host(ticket, [])
            except Exception:
                pass


@dataclasses.dataclass
class BoundKernel:
    """One kernel family bound to one call shape and math mode.

    `msl_source` names the CUDA source the family is built from (the reference
    keeps the emitted MSL text there, src/palladium/dispatch.py:90-108)."""

    spec: KernelSpec
    math_mode: int
    threadgroup: int | tuple[int, ...] | None = None
    msl_source: str = "palladium_b200/csrc/pd_kernels.cu"
    _in_sizes: list | None = dataclasses.field(default=None, compare=False, repr=False)
    _out_sizes: list | None = dataclasses.field(default=None, compare=False, repr=False)
    # Launches go through the library's slot pool (a stream and an event per call in flight), which
    # serialises what it must itself: no lock is held here, neither to launch nor to wait
    # (src/palladium/dispatch.py:121-127 holds one per kernel for launching).

    # ------------------------------------------------------------------ checks
    def _checked(self, arrays) -> list[np.ndarray]:
        spec = self.spec
        if len(arrays) != len(spec.inputs):
            raise DispatchError(f"kernel takes {len(spec.inputs)} arrays, got {len(arrays)}")
        out = []
        for i, (a, info) in enumerate(zip(arrays, spec.inputs)):
            arr = np.asarray(a)
            if arr.dtype != info.dtype:
                raise DispatchError(
                    f"argument {i}: dtype {arr.dtype} does not match the traced {info.dtype}; cast explicitly"
                )
            if arr.shape != info.array_shape:
                raise DispatchError(f"argument {i}: expected shape {info.array_shape}, got {arr.shape}")
            out.append(np.ascontiguousarray(arr))
        return out

    # ------------------------------------------------------------------ launch
    def launch(self, *arrays) -> PendingResult:
        """Upload, launch and start the read-back without blocking on the
        result.  The arrays are copied before this returns, so the caller may
        change them at once; any number of launches (up to the library's 64 slots)
        may be in flight, each on a stream of its own.  Thread-safe."""
        arrs = self._checked(arrays)
        _require_cuda()
        return self._submit([(a.ctypes.data, a.nbytes) for a in arrs], False)

    def _submit(self, inputs, on_device: bool) -> PendingResult:
        spec = self.spec
        if self._out_sizes is None:
            self._out_sizes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.outputs]
        out_host = None
        if sum(self._out_sizes) >= _DIRECT_OUTPUT_BYTES:
            # Large results download straight into fresh page-locked arrays (torch's caching host
            # allocator), which the returned NumPy arrays then view: no copy and no page faults
            # at the wait.  Small ones come back packed in one copy and are unpacked there.
            torch = _torch()
            out_host = [torch.empty(max(b, 1), dtype=torch.uint8, pin_memory=True) for b in self._out_sizes]
        ticket = _native.submit_host(spec.family.family_id, spec.params, self.math_mode, spec.grid, self.threadgroup,
                                     inputs, self._out_sizes,
                                     [t.data_ptr() for t in out_host] if out_host is not None else None, on_device)
        return PendingResult(spec.outputs, ticket=ticket, out_host=out_host)

    def __call__(self, *arrays):
        """Dispatch over `spec.grid` and return the outputs (NumPy)."""
        return self.launch(*arrays).wait()

    def pinned(self, *arrays) -> Callable[[], object]:
        """Upload `arrays` once; return a zero-argument callable that
        re-dispatches on the device-resident inputs.  Later mutation of the
        passed arrays is not observed (src/palladium/dispatch.py:230-255)."""
        arrs = self._checked(arrays)
        torch = _require_cuda()
        resident = [torch.from_numpy(a.reshape(-1).view(np.uint8).copy()).to("cuda", non_blocking=False)
                    if a.nbytes else torch.empty(1, dtype=torch.uint8, device="cuda") for a in arrs]
        torch.cuda.current_stream().synchronize()

        pointers = [(t.data_ptr(), a.nbytes) for t, a in zip(resident, arrs)]

        def call(_resident=resident):     # the default argument keeps the device copies alive with the callable
            return self._submit(pointers, True).wait()

        return call

    # ------------------------------------------------------------------ device-resident path
    def launch_device(self, inputs, outputs=None, stream=None, workspace=None):
        """Launch on torch CUDA tensors, stream-ordered, without any host
        synchronisation or copy.  `inputs`: one tensor per kernel input, holding
        exactly the bytes of the traced operand.  Returns the output tensors
        (allocated as uint8 byte buffers unless `outputs` is given).
        `workspace`: a uint8 CUDA tensor of at least `scratch_bytes` (see
        `pd_explain`) for the kernels' scratch, in place of the library's own
        per-stream pool -- a caller that records launches into a CUDA graph owns
        the memory the graph keeps pointing at this way."""
        torch = _require_cuda()
        spec = self.spec
        if len(inputs) != len(spec.inputs):
            raise DispatchError(f"kernel takes {len(spec.inputs)} arrays, got {len(inputs)}")
        if self._in_sizes is None:
            self._in_sizes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.inputs]
        if self._out_sizes is None:
            self._out_sizes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.outputs]
        in_bytes, out_bytes = self._in_sizes, self._out_sizes
        current = torch.cuda.current_device()
        check_device_tensors("argument", inputs, in_bytes, current)
        if stream is not None:
            raw_stream = stream.cuda_stream
        else:
            raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)   # the handle alone, without a Stream object
            raw_stream = raw(current) if raw is not None else torch.cuda.current_stream().cuda_stream
        if outputs is None:
            with torch.cuda.stream(stream if stream is not None else torch.cuda.current_stream()):
                outputs = [torch.empty(max(b, 1), dtype=torch.uint8, device="cuda") for b in out_bytes]
        elif len(outputs) != len(out_bytes):
            raise DispatchError(f"kernel produces {len(out_bytes)} arrays, got {len(outputs)} output tensors")
        else:
            # The kernel writes `out_bytes[i]` bytes from each pointer whatever the tensor's own
            # size or strides: a short, strided, host or other-device tensor must stop here.
            check_device_tensors("output", outputs, out_bytes, current)
        _native.launch(
            spec.family.family_id, spec.params, self.math_mode, spec.grid, self.threadgroup,
            [(t.data_ptr(), b) for t, b in zip(inputs, in_bytes)],
            [(t.data_ptr(), b) for t, b in zip(outputs, out_bytes)],
            stream=raw_stream,
            workspace=(workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else None,
        )
        return outputs


def check_device_tensors(what: str, tensors, nbytes, device_index: int) -> None:
    """Refuse, before any launch, a tensor the kernel could not safely read or
    write: the native call is given a pointer and the byte count of the traced
    operand, so the tensor must be on the launching CUDA device, contiguous, and
    hold exactly that many bytes."""
    for i, (t, b) in enumerate(zip(tensors, nbytes)):
        if not getattr(t, "is_cuda", False):
            raise DispatchError(f"{what} {i}: expected a CUDA tensor, got one on {getattr(t, 'device', 'the host')}")
        if not t.is_contiguous():
            raise DispatchError(f"{what} {i}: expected a contiguous tensor (a strided view cannot be passed by pointer)")
        have = t.numel() * t.element_size()
        if have != b:
            raise DispatchError(f"{what} {i}: expected {b} bytes, got {have}")
        index = getattr(t.device, "index", None)
        if index is not None and index != device_index:
            raise DispatchError(f"{what} {i}: tensor is on cuda:{index} but the launch runs on cuda:{device_index}")


def bind(spec: KernelSpec, msl_source: str | None = None, *, math_mode=MathMode.FAST,
         threadgroup: int | tuple[int, ...] | None = None) -> BoundKernel:
    """Bind a validated call to the native library.

    Mirrors `bind(spec, msl_source, math_mode=..., threadgroup=...)`
    (src/palladium/dispatch.py:258-314); `msl_source` is accepted for signature
    compatibility and ignored, because the kernels are precompiled.  Loading the
    library here makes a missing build fail at bind time, not at first launch."""
    _native.library()
    _dump_source(spec, math_mode)
    return BoundKernel(spec=spec, math_mode=math_mode_ordinal(math_mode), threadgroup=threadgroup)
