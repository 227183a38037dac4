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


@dataclasses.dataclass
class PendingResult:
    """A launched call whose kernels may still be executing.

    `wait()` blocks on the CUDA event recorded after the device-to-host copies
    and returns the outputs as NumPy arrays (a bare array for one output), the
    contract of src/palladium/dispatch.py:66-86."""

    event: object
    out_host: list
    out_infos: tuple

    def wait(self):
        self.event.synchronize()
        # A kernel whose bounded wait ran out recorded a code instead of computing: report it
        # rather than return fields that were never written (the eager call is blocking, like
        # mr_dispatch in the reference, so this is where its status surfaces).
        code = _native.device_status()
        if code:
            raise PalladiumError(f"device status {code}: a kernel's bounded wait ran out (a tile copy did not arrive "
                                 "within its limit); the outputs of this call are not valid")
        outs = tuple(
            host.numpy().view(info.dtype).reshape(info.array_shape) for host, info in zip(self.out_host, self.out_infos)
        )
        return outs[0] if len(outs) == 1 else outs


@dataclasses.dataclass
class BoundKernel:
    """One kernel family bound to one call shape and math mode.

    `msl_source` names the CUDA source the family is built from (the reference
    keeps the emitted MSL text there, src/palladium/dispatch.py:90-108)."""

    spec: KernelSpec
    math_mode: int
    threadgroup: int | tuple[int, ...] | None = None
    msl_source: str = "palladium_b200/csrc/pd_kernels.cu"
    _in_dev: list = dataclasses.field(default_factory=list, compare=False, repr=False)
    _in_host: list = dataclasses.field(default_factory=list, compare=False, repr=False)
    _last_pending: PendingResult | None = dataclasses.field(default=None, compare=False, repr=False)
    _stream: object = dataclasses.field(default=None, compare=False, repr=False)
    # Serialises upload-and-launch: concurrent launches share the input staging
    # buffers, and each launch waits out the previous one before overwriting
    # them.  Waiting on results stays unlocked (src/palladium/dispatch.py:121-127).
    _launch_lock: threading.Lock = dataclasses.field(default_factory=threading.Lock, compare=False, repr=False)

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

    def _ensure_stream(self, torch):
        if self._stream is None:
            self._stream = torch.cuda.Stream()
        return self._stream

    # ------------------------------------------------------------------ launch
    def _run(self, torch, in_dev: list, stream) -> PendingResult:
        """Launch on device inputs; copy the outputs into fresh pinned buffers."""
        spec = self.spec
        out_bytes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.outputs]
        with torch.cuda.stream(stream):
            out_dev = [torch.empty(max(b, 1), dtype=torch.uint8, device="cuda") for b in out_bytes]
            in_bytes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.inputs]
            _native.launch(
                spec.family.family_id, spec.params, self.math_mode, spec.grid, self.threadgroup,
                [(t.data_ptr(), b) for t, b in zip(in_dev, in_bytes)],
                [(t.data_ptr(), b) for t, b in zip(out_dev, out_bytes)],
                stream=stream.cuda_stream,
            )
            # Fresh per call: a caller may still hold the arrays of an earlier,
            # not yet waited-on result (src/palladium/dispatch.py:180-186).
            out_host = [torch.empty(b, dtype=torch.uint8, pin_memory=True) for b in out_bytes]
            for host, dev, b in zip(out_host, out_dev, out_bytes):
                if b:
                    host.copy_(dev[:b], non_blocking=True)
            event = torch.cuda.Event()
            event.record(stream)
        pending = PendingResult(event, out_host, spec.outputs)
        self._last_pending = pending
        return pending

    def launch(self, *arrays) -> PendingResult:
        """Upload, launch and start the read-back without blocking on the
        result.  Thread-safe: uploads are serialised per kernel, waits are not."""
        arrs = self._checked(arrays)
        torch = _require_cuda()
        with self._launch_lock:
            stream = self._ensure_stream(torch)
            if self._last_pending is not None:
                # The previous launch must be done reading the staging buffers.
                self._last_pending.event.synchronize()
            if not self._in_dev:
                for arr in arrs:
                    nbytes = max(arr.nbytes, 1)
                    self._in_host.append(torch.empty(nbytes, dtype=torch.uint8, pin_memory=True))
                    self._in_dev.append(torch.empty(nbytes, dtype=torch.uint8, device="cuda"))
            with torch.cuda.stream(stream):
                for arr, host, dev in zip(arrs, self._in_host, self._in_dev):
                    if arr.nbytes:
                        host.numpy()[: arr.nbytes] = arr.reshape(-1).view(np.uint8)
                        dev[: arr.nbytes].copy_(host[: arr.nbytes], non_blocking=True)
            return self._run(torch, self._in_dev, stream)

    def __call__(self, *arrays):
        """Dispatch over `spec.grid` and return the outputs (NumPy)."""
        return self.launch(*arrays).wait()

    def pinned(self, *arrays) -> Callable[[], object]:
        """Upload `arrays` once; return a zero-argument callable that
        re-dispatches on the device-resident inputs.  Later mutation of the
        passed arrays is not observed (src/palladium/dispatch.py:230-255)."""
        arrs = self._checked(arrays)
        torch = _require_cuda()
        stream = self._ensure_stream(torch)
        with torch.cuda.stream(stream):
            resident = [torch.from_numpy(a.reshape(-1).view(np.uint8).copy()).to("cuda", non_blocking=False)
                        if a.nbytes else torch.empty(1, dtype=torch.uint8, device="cuda") for a in arrs]
        stream.synchronize()

        def call():
            with self._launch_lock:
                pending = self._run(torch, resident, stream)
            return pending.wait()

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
        in_bytes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.inputs]
        out_bytes = [int(np.prod(info.array_shape)) * info.dtype.itemsize for info in spec.outputs]
        current = torch.cuda.current_device()
        check_device_tensors("argument", inputs, in_bytes, current)
        st = stream if stream is not None else torch.cuda.current_stream()
        if outputs is None:
            with torch.cuda.stream(st):
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
            stream=st.cuda_stream,
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
