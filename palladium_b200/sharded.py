"""Multi-GPU execution: one process per GPU, `torch.distributed` for the plumbing.

The reference has no multi-device code.  The three ways its kernels shard:

* ODE ensembles (RK4, adaptive, df32): trajectories are independent, so rank r
  integrates the contiguous slab `partition(n, world, r)`; no collective.
* GBM Monte Carlo: paths are independent and the RNG stream of a path is keyed
  by its *global* index (`path_offset`), so results do not depend on the number
  of ranks; the per-rank float64 sums (payoff, payoff^2) are combined with ONE
  all-reduce (NCCL over NVLink on GPUs).
* Gray-Scott: row slabs on a periodic ring of ranks.  Each rank keeps `halo`
  ghost rows above and below its owned rows; one exchange fills them from the
  neighbours' boundary rows (point-to-point sends; the remote rows land in the
  receiver's own memory before any kernel reads them), after which `halo` steps
  run without communication (step s updates rows [s, rows + 2*halo - s), the
  redundant ghost-row work replaces an exchange per step).  Per-cell arithmetic
  is unchanged, so the result equals the single-grid result bit for bit.
  With `push=True` the exchange moves into the compute kernel: the final launch
  of each call stores the boundary rows into the neighbours' ghost rows (peer
  memory mapped with CUDA IPC, plain stores over NVLink) and a one-element
  all-reduce orders the calls; measured on two B200s at 8192 x 8192 per GPU,
  102.4 us per step against 107.6 with point-to-point sends and 102.7 on one
  GPU alone.

The step / path functions are injectable so the host logic (partitioning,
exchange pattern, reduction) can be exercised by CPU ranks over gloo; the
defaults run the CUDA kernels.
"""

from __future__ import annotations

import dataclasses
from collections.abc import Callable

import numpy as np

__all__ = ["partition", "ensemble_indices", "run_ensemble", "GbmResult", "gbm_monte_carlo", "GrayScottSlab"]


def partition(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous slab [lo, hi) of n units for `rank`; sizes differ by at most 1."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    base, extra = divmod(int(n), world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _dist():
    import torch.distributed as dist

    return dist


def _world(group=None) -> tuple[int, int]:
    dist = _dist()
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


# ----------------------------------------------------------------------------- ODE ensembles
def ensemble_indices(n: int, world: int, rank: int, interleave: bool = False):
    """The trajectories rank `rank` integrates: the contiguous slab of
    `partition`, or every `world`-th trajectory starting at `rank` when
    `interleave` is set.  Interleaving evens out the cost per rank when the cost
    of a trajectory varies along the array (an adaptive solver over stiffness
    parameters stored in sorted order)."""
    if interleave:
        if world <= 0 or not 0 <= rank < world:
            raise ValueError(f"rank {rank} is not in a world of {world}")
        return slice(rank, int(n), world)
    lo, hi = partition(n, world, rank)
    return slice(lo, hi)


def run_ensemble(make_call: Callable, arrays, *, interleave: bool = False, gather: bool = False, group=None):
    """Integrate this rank's share of a per-trajectory ensemble.

    `arrays` are the full-length inputs (NumPy arrays or torch tensors, first
    axis = trajectory), identical on every rank; `make_call(n_local)` returns the
    call for `n_local` trajectories (a `cuda_call` / `cuda_call_jit` object, or any
    function of the local arrays when the host logic runs on CPU ranks).
    Trajectories are independent, so no data-path collective is needed; with
    `gather=True` the outputs of all ranks are all-gathered and put back in
    the original trajectory order, otherwise each rank returns its own share.
    Returns (outputs tuple, index slice of this rank's trajectories)."""
    import torch

    rank, world = _world(group)
    n = int(arrays[0].shape[0])
    idx = ensemble_indices(n, world, rank, interleave)
    local = []
    for a in arrays:
        part = a[idx]
        local.append(part.contiguous() if isinstance(part, torch.Tensor) else np.ascontiguousarray(part))
    n_local = int(local[0].shape[0])
    outs = make_call(n_local)(*local)
    outs = tuple(outs) if isinstance(outs, (tuple, list)) else (outs,)
    if not gather or world == 1:
        return outs, idx
    dist = _dist()
    cap = -(-n // world)              # the largest share; shorter shares are padded for the collective
    full = []
    for o in outs:
        was_numpy = not isinstance(o, torch.Tensor)
        t = torch.from_numpy(np.ascontiguousarray(o)) if was_numpy else o
        pad = torch.zeros((cap, *t.shape[1:]), dtype=t.dtype, device=t.device)
        pad[:n_local] = t
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad, group=group)
        whole = torch.empty((n, *t.shape[1:]), dtype=t.dtype, device=t.device)
        for r, part in enumerate(parts):
            ridx = ensemble_indices(n, world, r, interleave)
            count = len(range(*ridx.indices(n)))
            whole[ridx] = part[:count]
        full.append(whole.numpy() if was_numpy else whole)
    return tuple(full), idx


# ----------------------------------------------------------------------------- Monte Carlo
@dataclasses.dataclass
class GbmResult:
    price: float          # discounted mean payoff over ALL ranks' paths
    stderr: float         # its standard error
    n_total: int
    local_lo: int
    local_hi: int
    local_output: object  # this rank's per-path output (device tensor or array)
    sums: tuple[float, float]  # global (sum payoff, sum payoff^2)


_GBM_CALLS: dict = {}


def _cuda_gbm_paths(key, lo: int, n_local: int, constants: dict, math_mode, output: str):
    """Default path function: the CUDA kernel on this rank's GPU.  Returns
    (per-path output tensor, float64 tensor [sum payoff, sum payoff^2])."""
    import torch

    from . import cuda_call_jit, families, pl

    cache_key = (lo, n_local, output, tuple(sorted(constants.items())), str(math_mode), torch.cuda.current_device())
    call = _GBM_CALLS.get(cache_key)
    if call is None:
        fam = families.gbm_threefry(output=output, path_offset=lo, **constants)
        call = cuda_call_jit(fam, grid=(n_local,),
                             out_shape=(pl.ShapeDtypeStruct((n_local,), np.float32), pl.ShapeDtypeStruct((2,), np.float64)),
                             math_mode=math_mode)
        if len(_GBM_CALLS) >= 16:
            _GBM_CALLS.clear()
        _GBM_CALLS[cache_key] = call
    key_dev = torch.from_numpy(np.asarray(key, np.uint32).copy()).cuda()
    out, sums = call(key_dev)
    return out, sums


def gbm_monte_carlo(key, n_total: int, constants: dict, *, math_mode="fast", output: str = "terminal", group=None,
                    path_fn: Callable | None = None) -> GbmResult:
    """Price a European call over `n_total` GBM paths spread across the ranks of
    `group` (examples/03_sde_montecarlo.py:137-146 computes the same price from
    one device's payoffs).  `constants`: s0, strike, r, sigma, t, steps."""
    import torch

    dist = _dist()
    rank, world = _world(group)
    lo, hi = partition(n_total, world, rank)
    fn = path_fn or _cuda_gbm_paths
    out, sums = fn(key, lo, hi - lo, constants, math_mode, output)
    sums_t = sums if isinstance(sums, torch.Tensor) else torch.as_tensor(np.asarray(sums, np.float64))
    sums_t = sums_t.to(torch.float64).clone()
    if world > 1:
        dist.all_reduce(sums_t, op=dist.ReduceOp.SUM, group=group)
    s1, s2 = (float(v) for v in sums_t.cpu())
    disc = float(np.exp(-constants["r"] * constants["t"]))
    mean = s1 / n_total
    var = max(s2 / n_total - mean * mean, 0.0) * n_total / max(n_total - 1, 1)
    return GbmResult(price=disc * mean, stderr=disc * float(np.sqrt(var / n_total)), n_total=n_total, local_lo=lo,
                     local_hi=hi, local_output=out, sums=(s1, s2))


# ----------------------------------------------------------------------------- stencil
_SLAB_CALLS: dict = {}


def _cuda_slab_step(u, v, steps: int, halo: int, rows: int, cols: int, constants: dict, math_mode, out=None):
    """Default step function: `steps` (<= halo) stencil steps on a device slab."""
    from . import cuda_call_jit, families, pl

    key = (steps, halo, rows, cols, tuple(sorted(constants.items())), str(math_mode))
    call = _SLAB_CALLS.get(key)
    if call is None:
        shape = (rows + 2 * halo, cols)
        fam = families.gray_scott(steps=steps, halo=halo, **constants)
        call = cuda_call_jit(fam, grid=(rows, cols),
                             out_shape=(pl.ShapeDtypeStruct(shape, np.float32), pl.ShapeDtypeStruct(shape, np.float32)),
                             math_mode=math_mode)
        _SLAB_CALLS[key] = call
    return call.on_device(u, v, out=out)


class GrayScottSlab:
    """One rank's row slab of a periodic (rows_total x cols) Gray-Scott grid.

    Parameters
    ----------
    u, v : this rank's owned rows, shape (hi - lo, cols), as torch tensors on the
        rank's device (CUDA for the default step function).
    rows_total : global row count; this rank owns rows `partition(rows_total, world, rank)`.
    halo : ghost rows per side = steps advanced per exchange.  Measured on two
        B200s at 8192 x 8192 per GPU: 119 / 110 / 107 us per step for halo 4 / 8 /
        16 against 104 us on one GPU without any exchange -- the cost of an
        exchange is its fixed launch latency, so deeper halos amortise it.
    overlap : run the exchange on a second stream behind the interior rows
        (`_advance_overlapped`).  Correct and tested, but it measured no gain at
        any halo depth (the exchange is latency, not bandwidth), so it is off.
    push : the exchange from inside the compute kernel.  The slab's fields live in
        memory the neighbours have mapped (CUDA IPC); the final launch of every
        call stores the boundary rows to its own output and, from the same
        registers, into the neighbours' ghost rows over NVLink, and the only
        collective left is a one-element all-reduce that orders "everyone's call
        has finished" before the next call (nothing waits inside a kernel).  Two
        output sets alternate, so a neighbour never reads the set being written.
        CUDA step function only; the first call still fills the ghost rows with
        the point-to-point exchange.
    timeout, block_host : how long a rank waits for its neighbours in an exchange
        (seconds), and whether the host blocks in that wait.  With the host
        blocking (the default for CPU fields) a neighbour that left the stepping
        loop between calls ends the wait after `timeout` with a `DispatchError`
        naming the ranks that never arrived, instead of waiting forever.  For
        CUDA fields the default is a stream-ordered wait (the host runs ahead and
        the launch queue stays full); there the process group's own timeout bounds
        the wait, or pass `block_host=True` to get the bounded host wait.
    """

    def __init__(self, u, v, rows_total: int, *, halo: int = 4, constants: dict | None = None, math_mode="fast",
                 group=None, step_fn: Callable | None = None, overlap: bool = False, push: bool = False,
                 timeout: float = 120.0, block_host: bool | None = None):
        import torch

        if timeout <= 0:
            raise ValueError("timeout must be positive (seconds)")
        self.timeout = float(timeout)
        self.block_host = (not u.is_cuda) if block_host is None else bool(block_host)
        self.calls = 0
        self.overlap = overlap
        self.push = bool(push)
        if self.push and step_fn is not None:
            raise ValueError("push=True needs the CUDA step function (it stores into the neighbours' device memory)")
        self._comm = None
        self._out = None

        self.group = group
        self.rank, self.world = _world(group)
        self.lo, self.hi = partition(rows_total, self.world, self.rank)
        self.rows = self.hi - self.lo
        self.cols = int(u.shape[1])
        if tuple(u.shape) != (self.rows, self.cols) or tuple(v.shape) != (self.rows, self.cols):
            raise ValueError(f"rank {self.rank} owns rows [{self.lo}, {self.hi}): expected fields of shape "
                             f"{(self.rows, self.cols)}, got {tuple(u.shape)} and {tuple(v.shape)}")
        if halo < 1:
            raise ValueError("halo must be at least 1")
        if self.rows < halo:
            raise ValueError(f"a slab of {self.rows} rows cannot serve {halo} ghost rows to its neighbours")
        self.halo = halo
        self.constants = dict(constants or {})
        self.math_mode = math_mode
        self.step_fn = step_fn or _cuda_slab_step
        shape = (self.rows + 2 * halo, self.cols)
        self.u = torch.empty(shape, dtype=u.dtype, device=u.device)
        self.v = torch.empty(shape, dtype=v.dtype, device=v.device)
        self.u[halo:halo + self.rows] = u
        self.v[halo:halo + self.rows] = v
        self.up = (self.rank - 1) % self.world    # owns the rows above ours
        self.down = (self.rank + 1) % self.world  # owns the rows below ours
        self.exchanges = 0
        self.pushes = 0
        if self.push:
            self._setup_push()

    # -- exchange from inside the kernel ---------------------------------------------
    def _setup_push(self) -> None:
        """Move the fields into IPC-exportable allocations (two sets), trade the
        handles with the neighbours and map theirs."""
        import torch

        from . import _native

        shape = (self.rows + 2 * self.halo, self.cols)
        nbytes = shape[0] * shape[1] * 4
        if self.u.dtype != torch.float32:
            raise ValueError("push=True needs float32 fields")
        device = self.u.device

        class _Raw:   # a device allocation seen through the CUDA array interface
            def __init__(self, ptr):
                self.ptr = ptr
                self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (ptr, False), "version": 3,
                                                 "strides": None}

        self._raw, self._sets = [], []
        with torch.cuda.device(device):
            for _ in range(2):
                fields = []
                for _f in range(2):
                    raw = _Raw(_native.peer_alloc(nbytes))
                    self._raw.append(raw)
                    fields.append(torch.as_tensor(raw, device=device))
                self._sets.append(tuple(fields))
        self._sets[0][0].copy_(self.u)
        self._sets[0][1].copy_(self.v)
        self._sets[1][0].zero_()
        self._sets[1][1].zero_()
        self.u, self.v = self._sets[0]
        self._cur = 0
        self._ghosts_valid = False
        torch.cuda.synchronize(device)
        mine = (self.rows, [_native.peer_export(raw.ptr) for raw in self._raw])   # order: set0 u, set0 v, set1 u, set1 v
        if self.world == 1:
            everyone = [mine]
        else:
            dist = _dist()
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=self.group)
        self._opened: dict = {}

        def pointers(rank):
            if rank == self.rank:
                return [raw.ptr for raw in self._raw]
            if rank not in self._opened:
                with torch.cuda.device(device):
                    self._opened[rank] = [_native.peer_open(h) for h in everyone[rank][1]]
            return self._opened[rank]

        up_ptrs, down_ptrs = pointers(self.up), pointers(self.down)
        self._neighbours = [
            _native.GsNeighbours(up_ptrs[2 * k], up_ptrs[2 * k + 1], everyone[self.up][0],
                                 down_ptrs[2 * k], down_ptrs[2 * k + 1], everyone[self.down][0])
            for k in range(2)
        ]
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        if self.world > 1:
            _dist().barrier(group=self.group)   # every rank has mapped its neighbours before anyone pushes

    def _advance_push(self, k: int) -> None:
        import torch

        from . import _native
        from .math_mode import math_mode_ordinal

        if not self._ghosts_valid:
            self.exchange()                      # the first call: ghost rows from the initial state
        c = self.constants
        defaults = dict(du=0.16, dv=0.08, f=0.035, k=0.065, dt=1.0)
        defaults.update(c)
        params = _native.GrayScottParams(defaults["du"], defaults["dv"], defaults["f"], defaults["k"], defaults["dt"],
                                         k, self.rows, self.cols, self.halo)
        out = 1 - self._cur
        (u, v), (uo, vo) = self._sets[self._cur], self._sets[out]
        with torch.cuda.device(u.device):
            _native.gray_scott_slab_push(params, math_mode_ordinal(self.math_mode), u.data_ptr(), v.data_ptr(),
                                         uo.data_ptr(), vo.data_ptr(), self._neighbours[out],
                                         torch.cuda.current_stream().cuda_stream)
        if self.world > 1:
            # orders "every rank's call (and its stores into our ghost rows) has finished"
            # before anyone's next call reads them
            self._wait([_dist().all_reduce(self._flag, group=self.group, async_op=True)],
                       "the all-reduce that orders the calls of the in-kernel exchange")
        self._cur = out
        self.u, self.v = self._sets[out]
        self._ghosts_valid = True
        self.pushes += 1

    def close(self) -> None:
        """Unmap the neighbours' memory and free this slab's exportable allocations
        (push mode; call on every rank, after a barrier, when the slab is done)."""
        if not self.push or not getattr(self, "_raw", None):
            return
        import torch

        from . import _native

        torch.cuda.synchronize(self.u.device)
        self.u, self.v = self.u.clone(), self.v.clone()
        with torch.cuda.device(self.u.device):
            for ptrs in self._opened.values():
                for ptr in ptrs:
                    _native.peer_close(ptr)
            self._opened = {}
            if self.world > 1:
                _dist().barrier(group=self.group)    # nobody still maps our memory
            for raw in self._raw:
                _native.peer_free(raw.ptr)
        self._raw, self._sets = [], []
        self.push = False

    # -- communication ----------------------------------------------------------------
    def exchange(self) -> None:
        """Fill the ghost rows: our first `halo` owned rows go to the upper
        neighbour's bottom ghost rows, our last `halo` owned rows to the lower
        neighbour's top ghost rows (periodic ring)."""
        h, r = self.halo, self.rows
        self.exchanges += 1
        if self.world == 1:
            for f in (self.u, self.v):
                f[:h] = f[r:r + h]          # rows above row 0 are the last rows of the grid
                f[h + r:] = f[h:2 * h]      # rows below the last row are the first rows
            return
        if self.world == 2:
            # Both neighbours are the same rank: order the transfers explicitly so
            # the two messages per field cannot be matched crosswise.
            self._exchange_pairwise()
            return
        dist = _dist()
        ops, keep = [], []
        for f in (self.u, self.v):
            top_send = f[h:2 * h].contiguous()
            bot_send = f[r:r + h].contiguous()
            keep += [top_send, bot_send]
            ops += [dist.P2POp(dist.isend, top_send, self._global(self.up), group=self.group),
                    dist.P2POp(dist.isend, bot_send, self._global(self.down), group=self.group),
                    dist.P2POp(dist.irecv, f[:h], self._global(self.up), group=self.group),
                    dist.P2POp(dist.irecv, f[h + r:], self._global(self.down), group=self.group)]
        self._wait(dist.batch_isend_irecv(ops), "the halo exchange")

    def _wait(self, works, what: str) -> None:
        """Wait for the collective(s) of one exchange.  Host-blocking waits are
        bounded by `self.timeout`; when one runs out, the ranks that never
        reached this exchange are looked up and named."""
        self.calls += 1
        if not self.block_host:
            for work in works:
                work.wait()
            return
        from datetime import timedelta

        try:
            for work in works:
                work.wait(timedelta(seconds=self.timeout))
        except RuntimeError as exc:      # a timeout, or a connection a departed peer closed
            from .errors import DispatchError

            raise DispatchError(self._missing_ranks_message(what, exc)) from exc

    def _missing_ranks_message(self, what: str, exc: Exception) -> str:
        """Every rank whose wait ran out posts its rank under this slab's key in the
        job's key-value store; after a short grace period the ranks that posted
        nothing are the ones that are gone (left the loop, raised, or died)."""
        import time

        waited_on = sorted({self._global(self.up), self._global(self.down)})
        text = (f"rank {self.rank}: {what} with ranks {waited_on} did not complete within {self.timeout:g} s "
                f"(exchange {self.calls} of this slab)")
        try:
            store = _dist().distributed_c10d._get_default_store()
            me = self._global(self.rank)
            store.set(f"palladium_b200/slab_wait/{me}", str(self.calls))
            ranks = [self._global(r) for r in range(self.world)]
            missing = ranks
            deadline = time.monotonic() + min(2.0, self.timeout)
            while True:
                missing = [r for r in ranks if r != me and not store.check([f"palladium_b200/slab_wait/{r}"])]
                if not missing or time.monotonic() > deadline:
                    break
                time.sleep(0.05)
            if missing:
                text += f"; rank(s) {missing} never arrived (left the stepping loop or stopped)"
            else:
                text += "; every rank is waiting in an exchange, so the ranks disagree on the number of calls"
        except Exception:   # no store to ask: the neighbours waited on are all that is known
            pass
        return f"{text}: {exc}"

    def _exchange_pairwise(self) -> None:
        dist = _dist()
        h, r = self.halo, self.rows
        other = self._global(self.up)
        for f in (self.u, self.v):
            top_send = f[h:2 * h].contiguous()
            bot_send = f[r:r + h].contiguous()
            top_recv = f[:h]
            bot_recv = f[h + r:]
            # message 1: my top rows -> the other's bottom ghosts; message 2: my bottom rows -> its top ghosts
            first = [dist.P2POp(dist.isend, top_send, other, group=self.group),
                     dist.P2POp(dist.irecv, bot_recv, other, group=self.group)]
            self._wait(dist.batch_isend_irecv(first), "the halo exchange")
            second = [dist.P2POp(dist.isend, bot_send, other, group=self.group),
                      dist.P2POp(dist.irecv, top_recv, other, group=self.group)]
            self._wait(dist.batch_isend_irecv(second), "the halo exchange")

    def _global(self, group_rank: int) -> int:
        dist = _dist()
        if self.group is None:
            return group_rank
        return dist.get_global_rank(self.group, group_rank)

    # -- stepping ---------------------------------------------------------------------
    def advance(self, steps: int) -> None:
        """Advance the whole grid by `steps` steps: ceil(steps / halo) exchanges."""
        done = 0
        overlap = (self.step_fn is _cuda_slab_step and self.world > 1 and self.overlap
                   and self.rows >= 2 * self.halo + 1)
        while done < steps:
            k = min(self.halo, steps - done)
            if self.push:
                self._advance_push(k)
            elif overlap:
                self._advance_overlapped(k)
            else:
                self.exchange()
                self.u, self.v = self.step_fn(self.u, self.v, k, self.halo, self.rows, self.cols, self.constants,
                                              self.math_mode)
            done += k

    def _advance_overlapped(self, k: int) -> None:
        """One exchange + k steps with the exchange hidden behind the interior.

        The rows that do not depend on ghost rows -- the slab without its ghost
        rows, treated as a slab whose "ghosts" are our own boundary rows -- are
        advanced on the compute stream while the neighbours' rows travel on a
        second stream; the two boundary strips (3*halo rows each) follow once the
        ghost rows have landed.  All three launches write into one output slab;
        where their row ranges overlap they write identical values."""
        import torch

        h, R = self.halo, self.rows + 2 * self.halo
        main = torch.cuda.current_stream()
        if self._comm is None:
            self._comm = torch.cuda.Stream()
            self._out = None
        self._comm.wait_stream(main)            # the previous launch's outputs are our send buffers
        with torch.cuda.stream(self._comm):
            self.exchange()
        if self._out is None or self._out[0].shape != self.u.shape:
            self._out = (torch.empty_like(self.u), torch.empty_like(self.v))
        ou, ov = self._out
        args = (self.constants, self.math_mode)
        # interior: rows [h, R - h) as a slab of R - 4h owned rows
        _cuda_slab_step(self.u[h:R - h], self.v[h:R - h], k, h, R - 4 * h, self.cols, *args,
                        out=(ou[h:R - h], ov[h:R - h]))
        main.wait_stream(self._comm)            # ghost rows are in place
        _cuda_slab_step(self.u[:3 * h], self.v[:3 * h], k, h, h, self.cols, *args, out=(ou[:3 * h], ov[:3 * h]))
        _cuda_slab_step(self.u[R - 3 * h:], self.v[R - 3 * h:], k, h, h, self.cols, *args,
                        out=(ou[R - 3 * h:], ov[R - 3 * h:]))
        self._out = (self.u, self.v)            # ping-pong the two slabs
        self.u, self.v = ou, ov

    def owned(self):
        """This rank's owned rows of u and v (views)."""
        h = self.halo
        return self.u[h:h + self.rows], self.v[h:h + self.rows]
