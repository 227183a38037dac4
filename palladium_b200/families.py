"""Kernel families: what takes the place of a Pallas kernel function.

The reference traces an arbitrary Pallas function into a `KernelSpec` and emits
MSL for it (src/palladium/trace.py:117-178, src/palladium/emit/core.py:383-466).
This package has no emitter: the five integrator kernels are hand-written CUDA,
and `cuda_call(kernel, ...)` takes a *family descriptor* as its `kernel`
argument.  A descriptor names the family, carries the constants the reference
kernels close over as module globals (DT, STEPS, tolerances, ...), and checks
that the `grid` / `in_specs` / `out_specs` / `out_shape` of the call describe
the launch that family performs -- the same keywords, with the same meaning, a
user of the reference already writes for `metal_call`.

Two families are open-ended and compiled at run time, as the reference compiles
the MSL it emits: `custom_ode` (a right-hand side of the caller's inside the
library's RK4 or adaptive loop) and `source_kernel` (a complete CUDA kernel of
the caller's).

`trace(family, call_kwargs, *args)` produces the `KernelSpec` analogue: name,
grid, and one `BlockInfo` per operand.
"""

from __future__ import annotations

import ctypes
import dataclasses
from collections.abc import Callable, Sequence
from typing import Any

import numpy as np

from . import _native
from .errors import DispatchError, TraceError, UnsupportedPrimitiveError

__all__ = [
    "BlockInfo",
    "Family",
    "KernelSpec",
    "custom_ode",
    "gbm_pcg",
    "gbm_threefry",
    "gray_scott",
    "kepler_rk4_df32",
    "lv_rk4",
    "lv_rk4_df32",
    "source_kernel",
    "threefry_bits",
    "trace",
    "vdp_bs32",
    "vdp_cost_order",
]

F32 = np.dtype(np.float32)
U32 = np.dtype(np.uint32)
I32 = np.dtype(np.int32)
F64 = np.dtype(np.float64)


@dataclasses.dataclass(frozen=True)
class BlockInfo:
    """One operand of a traced call (src/palladium/trace.py:26-50)."""

    block_shape: tuple[int, ...]
    array_shape: tuple[int, ...]
    dtype: np.dtype


@dataclasses.dataclass(frozen=True)
class KernelSpec:
    """A validated call: the analogue of the reference's traced KernelSpec
    (src/palladium/trace.py:53-80) with the family in place of a jaxpr."""

    name: str
    family: "Family"
    grid: tuple[int, ...]
    inputs: tuple[BlockInfo, ...]
    outputs: tuple[BlockInfo, ...]
    params: ctypes.Structure

    @property
    def num_programs(self) -> int:
        return int(np.prod(self.grid)) if self.grid else 1


@dataclasses.dataclass(frozen=True)
class Family:
    """A hand-written kernel family plus the constants of one problem.

    `pallas_fn`, when given and JAX is installed, is the user's own Pallas
    kernel function for the same computation; `.interpret` then runs it through
    `pl.pallas_call(..., interpret=True)` exactly as the reference does."""

    name: str
    constants: dict[str, Any]
    pallas_fn: Callable | None = None

    @property
    def family_id(self) -> int:
        return _native.FAMILY_IDS[self.name]

    def __call__(self, *refs):
        raise UnsupportedPrimitiveError(
            f"{self.name} is a hand-written CUDA kernel family, not a Pallas function; "
            "pass it to palladium_b200.cuda_call instead of calling it"
        )


# ----------------------------------------------------------------------------- constructors
def lv_rk4(dt: float = 0.01, steps: int = 500, pallas_fn: Callable | None = None) -> Family:
    """Fixed-step RK4 Lotka-Volterra ensemble (examples/01_ode_ensembles.py:72-91).
    Call signature: grid=(N,), six (N,) float32 inputs x0, y0, a, b, c, d,
    two (N,) float32 outputs, or a single (N, 2) float32 output holding the
    final (x, y) pairs."""
    return Family("lv_rk4", dict(dt=float(dt), steps=int(steps)), pallas_fn)


def vdp_bs32(t1: float = 10.0, rtol: float = 1e-5, atol: float = 1e-7, dt0: float = 0.01,
             max_steps: int = 6000, pcoeff: float = 0.4, icoeff: float = 0.3, safety: float = 0.9,
             factor_min: float = 0.2, factor_max: float = 10.0, error_order: int = 3,
             pallas_fn: Callable | None = None) -> Family:
    """Adaptive Bogacki-Shampine 3(2) Van der Pol ensemble
    (examples/02_adaptive_lockstep.py:69-171; defaults from :20-32).
    grid=(N,), inputs x0, v0, mu.  The output layout follows `out_shape`:
    six float32 (N,) arrays t, x, v, steps, rejected, real; five (without
    `real`, tests/test_08_adaptive.py:33-142); or an (N, 2) float32 state plus
    int32 accepted and rejected counts."""
    return Family("vdp_bs32", dict(t1=float(t1), rtol=float(rtol), atol=float(atol), dt0=float(dt0),
                                   max_steps=int(max_steps), pcoeff=float(pcoeff), icoeff=float(icoeff),
                                   safety=float(safety), factor_min=float(factor_min),
                                   factor_max=float(factor_max), error_order=int(error_order)), pallas_fn)


_CHECKED_SOURCES: set = set()


_ODE_METHODS = {"rk4": 0, "bs32": 1, "dopri5": 2, "tsit5": 3}


def custom_ode(rhs: str, dim: int, nparam: int = 0, *, method: str = "rk4", dt: float = 0.01, steps: int = 500,
               t1: float = 10.0, rtol: float = 1e-5, atol: float = 1e-7, dt0: float = 0.01, max_steps: int = 6000,
               pcoeff: float = 0.4, icoeff: float = 0.3, safety: float = 0.9, factor_min: float = 0.2,
               factor_max: float = 10.0, error_order: int | None = None, check: bool = True,
               pallas_fn: Callable | None = None) -> Family:
    """An ensemble of independent systems y' = f(t, y, p) with a right-hand side
    of the caller's: the open end of the family set, where the reference lets a
    user write any Pallas function (and register lowering rules for what its
    emitter lacks, docs/extending.md:1-69).

    `rhs` is CUDA C: the statements of
    `void rhs(float t, const float* y, const float* p, float* dy)`, e.g.
    `"dy[0] = y[1]; dy[1] = (p[0] * (1.0f - y[0] * y[0])) * y[1] - y[0];"`.
    It is compiled at run time (NVRTC) under the flag set of the call's math
    mode and cached by source text, the way the reference compiles the MSL it
    emits on a cache miss (src/palladium/__init__.py:146-158).

    method="rk4": `steps` classic RK4 steps of `dt`; grid=(N,), inputs are the
    `dim` state arrays then the `nparam` parameter arrays, outputs the `dim`
    final states (all (N,) float32).  With the Lotka-Volterra right-hand side
    this reproduces `lv_rk4` bit for bit under MathMode.SAFE.
    method="bs32": adaptive Bogacki-Shampine 3(2) with the controller, counters
    and stall semantics of `vdp_bs32`; outputs t, the `dim` states, steps,
    rejected, real.
    method="dopri5" / "tsit5": the seven-stage 5(4) pairs of Dormand-Prince and of
    Tsitouras (what the reference's CPU comparison integrates with,
    benchmarks/bench_ensembles.py:88-118) under the same controller and with the
    same outputs.  `error_order` defaults to 3 for bs32 and 5 for these.

    With `check` (default) the source is compiled once here, without a GPU, so a
    faulty right-hand side raises EmitError where it is defined."""
    if method not in _ODE_METHODS:
        raise TraceError(f"custom_ode: method must be one of {sorted(_ODE_METHODS)}, got {method!r}")
    if error_order is None:
        error_order = 5 if method in ("dopri5", "tsit5") else 3
    if not isinstance(rhs, str) or not rhs.strip():
        raise TraceError("custom_ode: rhs must be a non-empty string of CUDA C statements")
    if not 1 <= int(dim) <= 8:
        raise TraceError(f"custom_ode: dim must lie in [1, 8], got {dim}")
    if not 0 <= int(nparam) <= 8:
        raise TraceError(f"custom_ode: nparam must lie in [0, 8], got {nparam}")
    fam = Family("custom_ode", dict(rhs=rhs, dim=int(dim), nparam=int(nparam), method=method, dt=float(dt),
                                    steps=int(steps), t1=float(t1), rtol=float(rtol), atol=float(atol),
                                    dt0=float(dt0), max_steps=int(max_steps), pcoeff=float(pcoeff),
                                    icoeff=float(icoeff), safety=float(safety), factor_min=float(factor_min),
                                    factor_max=float(factor_max), error_order=int(error_order)), pallas_fn)
    key = (rhs, int(dim), int(nparam), method)
    if check and key not in _CHECKED_SOURCES:
        _native.custom_ode_check(_custom_ode_params(fam.constants))
        _CHECKED_SOURCES.add(key)
    return fam


def _custom_ode_params(c: dict) -> "_native.CustomOdeParams":
    return _native.CustomOdeParams(c["rhs"].encode(), c["dim"], c["nparam"], _ODE_METHODS[c["method"]],
                                   c["dt"], c["steps"], c["t1"], c["rtol"], c["atol"], c["dt0"], c["pcoeff"],
                                   c["icoeff"], c["safety"], c["factor_min"], c["factor_max"], c["error_order"],
                                   c["max_steps"])


def source_kernel(source: str, function_name: str, check: bool = True) -> Family:
    """A complete kernel of your own as CUDA C source: what `metal_call` hands
    its runtime as emitted MSL plus an entry-point name
    (src/palladium/dispatch.py:286-292), written by hand here because there is
    no Pallas-to-CUDA emitter.

    The kernel is declared
    `extern "C" __global__ void name(T0* b0, ..., Tk* bk, long long gx, long long gy, long long gz)`:
    one pointer per array in call order (inputs, then the outputs of
    `out_shape`), then the extents of `grid`.  One thread runs per grid point,
    rounded up to whole blocks: return when `PD_THREAD_X >= gx` (and likewise
    `PD_THREAD_Y`, `PD_THREAD_Z`).  `pd_math.h` (Threefry, df32, `pd_powf`) is
    in scope.  Compiled at run time under the call's math mode, cached by
    source; array shapes and dtypes are whatever the call passes, unchecked
    against the kernel, as with hand-written MSL."""
    if not isinstance(source, str) or not source.strip():
        raise TraceError("source_kernel: source must be a non-empty string of CUDA C")
    if not isinstance(function_name, str) or not function_name.isidentifier() or len(function_name) > 63:
        raise TraceError(f"source_kernel: function_name must be a C identifier of at most 63 characters, "
                         f"got {function_name!r}")
    fam = Family("source", dict(source=source, function_name=function_name))
    key = ("source", source, function_name)
    if check and key not in _CHECKED_SOURCES:
        _native.source_kernel_check(_native.SourceKernelParams(source.encode(), function_name.encode()))
        _CHECKED_SOURCES.add(key)
    return fam


def vdp_cost_order(x0, v0, mu, *, pilot_rtol: float = 1e-3, pilot_atol: float = 1e-5, **constants):
    """A hand-out order for `vdp_bs32` from a pilot run at a looser tolerance.

    The adaptive kernel's run time ends with the trajectories that happen to be
    both long and late in the queue: each attempt of a lone trajectory costs its
    full dependent latency, so a 7500-attempt member started last adds
    milliseconds.  Handing out the trajectories by decreasing cost removes that
    tail -- with the true costs, 15.8 -> 13.7 ms at 2^20 trajectories (RELAXED) --
    and `vdp_bs32` takes such an order as an optional fourth operand (int32, a
    permutation of 0..N-1; results do not depend on it).  Use it when the costs
    are known, e.g. from an earlier solve of the same ensemble.

    This helper estimates them with a pilot run.  Measured, that does not pay:
    the pilot's step pattern predicts the tight-tolerance count only loosely
    (run 15.0 ms instead of 15.8, plus 0.8 ms for the pilot), so it is here for
    completeness rather than speed.  Takes and returns torch CUDA tensors."""
    import torch

    from .ffi import cuda_call_jit
    from .pl import ShapeDtypeStruct

    n = int(x0.shape[0])
    cfg = dict(constants)
    cfg.update(rtol=pilot_rtol, atol=pilot_atol)
    pilot = cuda_call_jit(vdp_bs32(**cfg), grid=(n,),
                          out_shape=(ShapeDtypeStruct((n, 2), np.float32), ShapeDtypeStruct((n,), np.int32),
                                     ShapeDtypeStruct((n,), np.int32)), math_mode="fast")
    _, accepted, rejected = pilot(x0, v0, mu)
    return torch.argsort(accepted + rejected, descending=True).to(torch.int32)


def gbm_threefry(s0: float = 100.0, strike: float = 105.0, r: float = 0.03, sigma: float = 0.2, t: float = 1.0,
                 steps: int = 256, output: str = "payoff", path_offset: int = 0,
                 pallas_fn: Callable | None = None) -> Family:
    """GBM European call paths with in-kernel Threefry (examples/03_sde_montecarlo.py:97-119;
    defaults from :30-32).  grid=(N,), one (2,) uint32 input (key data), one (N,)
    float32 output: the payoff max(S_T - K, 0) (`output="payoff"`, the reference)
    or the terminal price S_T (`output="terminal"`).  An optional second output
    of shape (2,) float64 receives (sum payoff, sum payoff^2)."""
    if output not in ("payoff", "terminal"):
        raise TraceError(f"gbm_threefry: output must be 'payoff' or 'terminal', got {output!r}")
    return Family("gbm_threefry", dict(s0=float(s0), strike=float(strike), r=float(r), sigma=float(sigma),
                                       t=float(t), steps=int(steps), output=output,
                                       path_offset=int(path_offset)), pallas_fn)


def gbm_pcg(s0: float = 100.0, strike: float = 105.0, r: float = 0.03, sigma: float = 0.2, t: float = 1.0,
            steps: int = 256, output: str = "payoff", path_offset: int = 0) -> Family:
    """The reference's hand-written GBM kernel (`GBM_MSL`, examples/03_sde_montecarlo.py:34-70):
    same model as `gbm_threefry` with the cheap `pcg_hash` counter RNG, one hash
    per uniform.  grid=(N,), no inputs, one (N,) float32 output (payoff or
    terminal price) and an optional (2,) float64 output of payoff sums."""
    if output not in ("payoff", "terminal"):
        raise TraceError(f"gbm_pcg: output must be 'payoff' or 'terminal', got {output!r}")
    return Family("gbm_pcg", dict(s0=float(s0), strike=float(strike), r=float(r), sigma=float(sigma), t=float(t),
                                  steps=int(steps), output=output, path_offset=int(path_offset)))


def gray_scott(du: float = 0.16, dv: float = 0.08, f: float = 0.035, k: float = 0.065, dt: float = 1.0,
               steps: int = 1, halo: int = 0, pallas_fn: Callable | None = None) -> Family:
    """Gray-Scott 5-point stencil (examples/04_reaction_diffusion.py:61-74; constants :35).
    grid=(rows, cols), inputs u, v and outputs u', v' of shape (rows, cols)
    float32.  `steps` > 1 runs that many steps inside one call with the fields
    resident on the device (the reference's ping-pong loop, :99-107).
    `halo` > 0 treats the arrays as a row slab of shape (rows + 2*halo, cols)
    with ghost rows that the caller fills; at most `halo` steps per call."""
    return Family("gray_scott", dict(du=float(du), dv=float(dv), f=float(f), k=float(k), dt=float(dt),
                                     steps=int(steps), halo=int(halo)), pallas_fn)


def lv_rk4_df32(dt: float = 0.01, steps: int = 500) -> Family:
    """RK4 Lotka-Volterra in df32 compensated arithmetic
    (examples/05_df32_precision.py:27-80).  Same signature as `lv_rk4`."""
    return Family("lv_rk4_df32", dict(dt=float(dt), steps=int(steps)))


def kepler_rk4_df32(dt: float = 1e-3, gm: float = 1.0, steps: int = 1000) -> Family:
    """RK4 two-body orbits in df32.  grid=(N,), eight (N,) float32 inputs
    (x, y, vx, vy as hi/lo pairs) and eight outputs of the same layout."""
    return Family("kepler_rk4_df32", dict(dt=float(dt), gm=float(gm), steps=int(steps)))


def threefry_bits(op: str = "bits", count: int = 1) -> Family:
    """The RNG primitives on their own (src/palladium/emit/rules.py:168-201):
    op "bits": (N,) uint32 = random_bits(key, (N,)); "uniform": (N,) float32;
    "fold_in": inputs key and (M,) uint32 data, output (M, 2) uint32 key data;
    "fold_uniform": (G, count) float32, row g = uniform(fold_in(key, g), (count,));
    "pcg": (N,) uint32 = pcg_hash(i), the hash of examples/03_sde_montecarlo.py:38-43
    (the key input is ignored)."""
    ops = {"bits": 0, "uniform": 1, "fold_in": 2, "fold_uniform": 3, "pcg": 4}
    if op not in ops:
        raise TraceError(f"threefry_bits: op must be one of {sorted(ops)}, got {op!r}")
    return Family("threefry_bits", dict(op=op, op_code=ops[op], count=int(count)))


# ----------------------------------------------------------------------------- tracing
def _shape_dtype(x) -> tuple[tuple[int, ...], np.dtype]:
    shape = getattr(x, "shape", None)
    dtype = getattr(x, "dtype", None)
    if shape is None or dtype is None:
        arr = np.asarray(x)
        shape, dtype = arr.shape, arr.dtype
    try:
        dtype = np.dtype(dtype)
    except TypeError:
        # a torch dtype: "torch.float32" -> float32
        dtype = np.dtype(str(dtype).rsplit(".", 1)[-1])
    return tuple(int(s) for s in shape), dtype


def _as_list(x) -> list:
    if x is None:
        return []
    if isinstance(x, (list, tuple)):
        return list(x)
    return [x]


def _check_specs(what: str, specs, expected_blocks: Sequence[tuple[tuple[int, ...], Callable]], grid) -> None:
    """Validate in_specs / out_specs against the block shapes and index maps the
    family implements.  A spec of None (or a missing list) is accepted: Pallas
    then defaults to whole-array blocks, which the fixed kernels do not depend on."""
    specs = _as_list(specs)
    if not specs:
        return
    if len(specs) != len(expected_blocks):
        raise TraceError(f"{what} has {len(specs)} entries, the kernel family takes {len(expected_blocks)}")
    probes = [tuple(0 for _ in grid), tuple(max(g - 1, 0) for g in grid)]
    for i, (spec, (block, index_map)) in enumerate(zip(specs, expected_blocks)):
        if spec is None:
            continue
        got_block = getattr(spec, "block_shape", None)
        if got_block is not None and tuple(int(b) for b in got_block) != tuple(block):
            raise TraceError(f"{what}[{i}]: block shape {tuple(got_block)} is not the {tuple(block)} this family uses")
        got_map = getattr(spec, "index_map", None)
        if got_map is not None:
            for probe in probes:
                try:
                    got = tuple(int(v) for v in got_map(*probe))
                except Exception as exc:  # a map of the wrong arity, most likely
                    raise TraceError(f"{what}[{i}]: index_map could not be evaluated at {probe}: {exc}") from None
                want = tuple(int(v) for v in index_map(*probe))
                if got != want:
                    raise TraceError(f"{what}[{i}]: index_map{probe} = {got}, this family needs {want}")


def _check_args(args, inputs: Sequence[BlockInfo]) -> None:
    if not args:
        return
    if len(args) != len(inputs):
        raise TraceError(f"kernel takes {len(inputs)} arrays, got {len(args)}")
    for i, (a, info) in enumerate(zip(args, inputs)):
        shape, dtype = _shape_dtype(a)
        if shape != info.array_shape:
            raise TraceError(f"argument {i}: shape {shape} does not match the {info.array_shape} implied by grid")
        if dtype != info.dtype:
            raise DispatchError(
                f"argument {i}: dtype {dtype} does not match the traced {info.dtype}; cast explicitly"
            )


def _out_structs(out_shape) -> list[tuple[tuple[int, ...], np.dtype]]:
    if out_shape is None:
        raise TraceError("out_shape is required")
    return [_shape_dtype(o) for o in _as_list(out_shape)]


def _per_item(n: int):
    return ((1,), lambda i: (i,))


def trace(family: Family, call_kwargs: dict[str, Any], *args) -> KernelSpec:
    """Validate a `pallas_call`-shaped call against a family; returns the spec.

    Raises TraceError when grid / specs / out_shape / argument shapes do not
    describe a launch of that family (the reference raises TraceError when a
    pallas_call cannot be traced, src/palladium/trace.py:83-99,139-166)."""
    if not isinstance(family, Family):
        raise UnsupportedPrimitiveError(
            "cuda_call needs a kernel family from palladium_b200.families (there is no "
            f"Pallas-to-CUDA emitter); got {type(family).__name__}"
        )
    unknown = set(call_kwargs) - {"grid", "in_specs", "out_specs", "out_shape", "name", "interpret", "debug",
                                  "input_output_aliases", "compiler_params", "cost_estimate", "grid_spec"}
    if unknown:
        raise TraceError(f"unsupported pallas_call keywords: {sorted(unknown)}")
    if call_kwargs.get("grid_spec") is not None:
        raise TraceError("grid_spec (scalar prefetch) is not supported; pass grid / in_specs / out_specs")
    if call_kwargs.get("input_output_aliases"):
        raise TraceError("input_output_aliases is not supported")
    grid = call_kwargs.get("grid")
    grid = (int(grid),) if isinstance(grid, (int, np.integer)) else tuple(int(g) for g in (grid or ()))
    outs = _out_structs(call_kwargs.get("out_shape"))
    c = family.constants
    name = family.name

    def vec(n, dtype=F32):
        return BlockInfo((1,), (n,), dtype)

    if name in ("lv_rk4", "lv_rk4_df32"):
        if len(grid) != 1:
            raise TraceError(f"{name}: grid must be (N,), got {grid}")
        n = grid[0]
        inputs = tuple(vec(n) for _ in range(6))
        outputs = tuple(vec(n) for _ in range(2))
        blocks_in = [_per_item(n)] * 6
        blocks_out = [_per_item(n)] * 2
        if name == "lv_rk4" and len(outs) == 1:
            # the final state as one (N, 2) array of (x, y) pairs
            outputs = (BlockInfo((1, 2), (n, 2), F32),)
            blocks_out = [((1, 2), lambda i: (i, 0))]
        if name == "lv_rk4":
            params = _native.LvRk4Params(c["dt"], c["steps"])
        else:
            params = _native.LvRk4Df32Params(c["dt"], c["steps"])
    elif name == "vdp_bs32":
        if len(grid) != 1:
            raise TraceError(f"{name}: grid must be (N,), got {grid}")
        n = grid[0]
        inputs = tuple(vec(n) for _ in range(3))
        blocks_in = [_per_item(n)] * 3
        if len(args) == 4 or len(_as_list(call_kwargs.get("in_specs"))) == 4:
            # optional fourth operand: the order in which the work queue hands out the
            # trajectories, a permutation of 0..N-1 (see `vdp_cost_order`)
            inputs = inputs + (vec(n, I32),)
            blocks_in = blocks_in + [_per_item(n)]
        if len(outs) == 6:
            layout, outputs, blocks_out = 0, tuple(vec(n) for _ in range(6)), [_per_item(n)] * 6
        elif len(outs) == 5:
            layout, outputs, blocks_out = 1, tuple(vec(n) for _ in range(5)), [_per_item(n)] * 5
        elif len(outs) == 3:
            layout = 2
            outputs = (BlockInfo((1, 2), (n, 2), F32), vec(n, I32), vec(n, I32))
            blocks_out = [((1, 2), lambda i: (i, 0)), _per_item(n), _per_item(n)]
        else:
            raise TraceError(f"{name}: out_shape must list 6, 5 or 3 outputs, got {len(outs)}")
        params = _native.VdpBs32Params(c["t1"], c["rtol"], c["atol"], c["dt0"], c["pcoeff"], c["icoeff"],
                                       c["safety"], c["factor_min"], c["factor_max"], c["error_order"],
                                       c["max_steps"], layout)
    elif name in ("gbm_threefry", "gbm_pcg"):
        if len(grid) != 1:
            raise TraceError(f"{name}: grid must be (N,), got {grid}")
        n = grid[0]
        if name == "gbm_threefry":
            inputs = (BlockInfo((2,), (2,), U32),)
            blocks_in = [((2,), lambda i: (0,))]
        else:
            inputs, blocks_in = (), []
        outputs = (vec(n),)
        blocks_out = [_per_item(n)]
        if len(outs) == 2:
            outputs = outputs + (BlockInfo((2,), (2,), F64),)
            blocks_out = blocks_out + [((2,), lambda i: (0,))]
        elif len(outs) != 1:
            raise TraceError(f"{name}: out_shape must list 1 or 2 outputs, got {len(outs)}")
        params = _native.GbmParams(c["s0"], c["strike"], c["r"], c["sigma"], c["t"], c["steps"], c["path_offset"],
                                   0 if c["output"] == "payoff" else 1)
    elif name == "gray_scott":
        if len(grid) != 2:
            raise TraceError(f"{name}: grid must be (rows, cols), got {grid}")
        rows, cols = grid
        shape = (rows + 2 * c["halo"], cols)
        inputs = tuple(BlockInfo(shape, shape, F32) for _ in range(2))
        outputs = tuple(BlockInfo(shape, shape, F32) for _ in range(2))
        blocks_in = [(shape, lambda i, j: (0, 0))] * 2
        blocks_out = [(shape, lambda i, j: (0, 0))] * 2
        params = _native.GrayScottParams(c["du"], c["dv"], c["f"], c["k"], c["dt"], c["steps"], rows, cols, c["halo"])
    elif name == "kepler_rk4_df32":
        if len(grid) != 1:
            raise TraceError(f"{name}: grid must be (N,), got {grid}")
        n = grid[0]
        inputs = tuple(vec(n) for _ in range(8))
        outputs = tuple(vec(n) for _ in range(8))
        blocks_in = [_per_item(n)] * 8
        blocks_out = [_per_item(n)] * 8
        params = _native.KeplerRk4Df32Params(c["dt"], c["gm"], c["steps"])
    elif name == "custom_ode":
        if len(grid) != 1:
            raise TraceError(f"{name}: grid must be (N,), got {grid}")
        n = grid[0]
        n_in = c["dim"] + c["nparam"]
        n_out = c["dim"] if c["method"] == "rk4" else c["dim"] + 4
        inputs = tuple(vec(n) for _ in range(n_in))
        outputs = tuple(vec(n) for _ in range(n_out))
        blocks_in = [_per_item(n)] * n_in
        blocks_out = [_per_item(n)] * n_out
        params = _custom_ode_params(c)
    elif name == "source":
        if not 1 <= len(grid) <= 3:
            raise TraceError(f"{name}: grid must have 1 to 3 dimensions, got {grid}")
        # the kernel defines its own operands: take them as the call gives them
        inputs = tuple(BlockInfo(shape, shape, dtype) for shape, dtype in (_shape_dtype(a) for a in args))
        outputs = tuple(BlockInfo(shape, shape, dtype) for shape, dtype in outs)
        blocks_in = blocks_out = None
        params = _native.SourceKernelParams(c["source"].encode(), c["function_name"].encode())
    elif name == "threefry_bits":
        if len(grid) != 1:
            raise TraceError(f"{name}: grid must be (N,), got {grid}")
        n = grid[0]
        key = BlockInfo((2,), (2,), U32)
        op = c["op"]
        if op in ("bits", "pcg"):
            inputs, outputs = (key,), (vec(n, U32),)
        elif op == "uniform":
            inputs, outputs = (key,), (vec(n),)
        elif op == "fold_in":
            inputs, outputs = (key, vec(n, U32)), (BlockInfo((1, 2), (n, 2), U32),)
        else:
            inputs, outputs = (key,), (BlockInfo((1, c["count"]), (n, c["count"]), F32),)
        blocks_in = blocks_out = None
        params = _native.ThreefryParams(c["op_code"], c["count"])
    else:
        raise UnsupportedPrimitiveError(f"no CUDA kernel family named {name!r}")

    if len(outs) != len(outputs):
        raise TraceError(f"{name}: out_shape lists {len(outs)} outputs, the kernel family produces {len(outputs)}")
    for i, ((shape, dtype), info) in enumerate(zip(outs, outputs)):
        if shape != info.array_shape or dtype != info.dtype:
            raise TraceError(
                f"{name}: out_shape[{i}] is {shape} {dtype}, the kernel family produces "
                f"{info.array_shape} {info.dtype} for grid {grid}"
            )
    if blocks_in is not None:
        _check_specs("in_specs", call_kwargs.get("in_specs"), blocks_in, grid)
        _check_specs("out_specs", call_kwargs.get("out_specs"), blocks_out, grid)
    _check_args(args, inputs)
    return KernelSpec(name=f"palladium_{name}", family=family, grid=grid, inputs=inputs, outputs=outputs, params=params)
