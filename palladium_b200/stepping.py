"""Device-resident stepping: many launches of one call with the state kept on
the GPU, one wait at the end.

The reference's stencil example drives its kernel this way by hand: two buffer
pairs on the device, one dispatch per step appended to a single batch with the
pairs swapped, one commit, one wait, and `batch.gpu_time` for the device-side
duration (examples/04_reaction_diffusion.py:92-109); its `launch()` / `wait()`
pair is the general form (src/palladium/dispatch.py:129-194).  `Stepper` is that
pattern as an object, for any call whose leading outputs are the next call's
leading inputs (the Gray-Scott fields, a df32 orbit state, the (x, y) state of
an ODE ensemble whose parameters stay fixed).
"""

from __future__ import annotations

from collections.abc import Sequence

import numpy as np

from .dispatch import BoundKernel, _require_cuda
from .errors import DispatchError

__all__ = ["Stepper"]


class Stepper:
    """Keeps a call's operands on the device and re-launches it in place.

    Parameters
    ----------
    call : CudaCallable or FfiCallable
        The call to repeat (e.g. `cuda_call(families.gray_scott(steps=4), ...)`:
        every launch then advances four steps).
    *arrays : numpy arrays
        Initial inputs, uploaded once.
    feedback : sequence of int, optional
        `feedback[k]` is the input slot that output k feeds for the next launch;
        by default output k feeds input k.  Inputs that no output feeds keep
        their initial values (per-trajectory parameters).
    """

    def __init__(self, call, *arrays, feedback: Sequence[int] | None = None):
        torch = _require_cuda()
        arrs = [np.ascontiguousarray(np.asarray(a)) for a in arrays]
        self._bound: BoundKernel = self._bind(call, arrs)
        spec = self._bound.spec
        self._bound._checked(arrs)
        n_out = len(spec.outputs)
        self._feedback = list(range(n_out)) if feedback is None else [int(i) for i in feedback]
        if len(self._feedback) != n_out:
            raise DispatchError(f"feedback must name one input slot per output ({n_out}), got {len(self._feedback)}")
        for k, slot in enumerate(self._feedback):
            if not 0 <= slot < len(spec.inputs):
                raise DispatchError(f"feedback[{k}] = {slot} is not an input slot")
            a, b = spec.outputs[k], spec.inputs[slot]
            if a.array_shape != b.array_shape or a.dtype != b.dtype:
                raise DispatchError(f"output {k} ({a.array_shape} {a.dtype}) cannot feed input {slot} "
                                    f"({b.array_shape} {b.dtype})")
        self._stream = torch.cuda.Stream()
        with torch.cuda.stream(self._stream):
            self._inputs = [torch.from_numpy(a.reshape(-1).view(np.uint8).copy()).cuda() if a.nbytes
                            else torch.empty(1, dtype=torch.uint8, device="cuda") for a in arrs]
            sizes = [max(int(np.prod(o.array_shape)) * o.dtype.itemsize, 1) for o in spec.outputs]
            # two output sets: a launch never writes the buffers it reads
            self._spare = [[torch.empty(s, dtype=torch.uint8, device="cuda") for s in sizes] for _ in range(2)]
            # The kernels' scratch (ping-pong fields of a multi-step stencil call, queue heads, partial
            # sums) belongs to this object rather than to the library's per-stream pool: a captured
            # graph keeps the pointer, and the pool may free and re-allocate its buffer when another
            # call on a stream with the same handle needs more.
            from . import _native

            info = _native.explain(spec.family.family_id, spec.params, self._bound.math_mode, spec.grid,
                                   self._bound.threadgroup)
            self._workspace = (torch.empty(int(info.scratch_bytes) + 256, dtype=torch.uint8, device="cuda")
                               if info.scratch_bytes > 0 else None)
        self._which = 0
        self._outputs = None
        self._start = torch.cuda.Event(enable_timing=True)
        self._end = torch.cuda.Event(enable_timing=True)
        self._timed = False
        self._graph = None
        self._graph_which = 0
        self.launches = 0

    def _aligned_workspace(self):
        """The workspace from its first 256-byte boundary on (the native call requires that alignment)."""
        if self._workspace is None:
            return None
        offset = (-self._workspace.data_ptr()) % 256
        return self._workspace[offset:]

    @staticmethod
    def _bind(call, arrs) -> BoundKernel:
        if hasattr(call, "_bound"):            # CudaCallable
            return call._bound(arrs)
        if hasattr(call, "_entry"):            # FfiCallable
            return call._entry(tuple((a.shape, a.dtype.name) for a in arrs))[1]
        raise DispatchError("Stepper needs a call built by cuda_call or cuda_call_jit")

    def advance(self, launches: int = 1, graph: bool = False) -> "Stepper":
        """Enqueue `launches` launches, each consuming the previous one's
        outputs; returns without waiting.

        graph=True replays the launches from a CUDA graph: the first call
        captures a unit of two launches (after which the ping-pong buffers are
        back in the same roles) and every unit after that costs one graph launch
        instead of two trips through the launch path.  Worth it when a launch is
        shorter than its launch overhead (small grids, few steps per launch)."""
        torch = _require_cuda()
        launches = int(launches)
        if graph and launches >= 4:
            launches = self._advance_graph(launches)
        with torch.cuda.stream(self._stream):
            if not self._timed:
                self._start.record(self._stream)
                self._timed = True
            for _ in range(launches):
                # Alternate between the two output sets: after this launch the fed
                # inputs alias set `which`, so the next launch must write the other.
                outs = self._spare[self._which]
                self._bound.launch_device(self._inputs, outs, stream=self._stream, workspace=self._aligned_workspace())
                for k, slot in enumerate(self._feedback):
                    self._inputs[slot] = outs[k]
                self._which = 1 - self._which
                self._outputs = outs
                self.launches += 1
            self._end.record(self._stream)
        return self

    def _advance_graph(self, launches: int) -> int:
        """Run as many two-launch units as fit from the captured graph; returns
        the launches left over for the eager path."""
        torch = _require_cuda()
        if self.launches < 2:
            # two eager launches first: every lazily created resource exists before the
            # capture (scratch, kernel attributes) and the fed inputs alias an output set
            self.advance(2)
            launches -= 2
        if self._graph is not None and self._which != self._graph_which:
            # the captured unit reads and writes fixed buffers: realign the ping-pong
            # phase with one eager launch before replaying it
            self.advance(1)
            launches -= 1
        units = launches // 2
        if units == 0:
            return launches
        if self._graph is None:
            self._graph_which = self._which
            self._stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self._stream):
                for _ in range(2):
                    outs = self._spare[self._which]
                    self._bound.launch_device(self._inputs, outs, stream=self._stream, workspace=self._aligned_workspace())
                    for k, slot in enumerate(self._feedback):
                        self._inputs[slot] = outs[k]
                    self._which = 1 - self._which
                    self._outputs = outs
            self._graph = g
        with torch.cuda.stream(self._stream):
            if not self._timed:
                self._start.record(self._stream)
                self._timed = True
            for _ in range(units):
                self._graph.replay()
            self._end.record(self._stream)
        self.launches += 2 * units
        return launches - 2 * units

    def wait(self) -> "Stepper":
        self._end.synchronize()
        return self

    @property
    def gpu_time(self) -> float:
        """Seconds the device spent between the first `advance` and the last
        launch so far (the analogue of `batch.gpu_time`)."""
        if not self._timed:
            return 0.0
        self._end.synchronize()
        return self._start.elapsed_time(self._end) / 1e3

    def read(self):
        """Wait, then return the latest outputs as NumPy arrays."""
        if self._outputs is None:
            raise DispatchError("nothing has been launched yet")
        self.wait()
        spec = self._bound.spec
        outs = []
        for t, info in zip(self._outputs, spec.outputs):
            nbytes = int(np.prod(info.array_shape)) * info.dtype.itemsize
            outs.append(t[:nbytes].cpu().numpy().view(info.dtype).reshape(info.array_shape))
        return outs[0] if len(outs) == 1 else tuple(outs)
