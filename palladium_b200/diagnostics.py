"""Kernel diagnostics: launch geometry for a validated call.

Mirrors the reference's `KernelDiagnostics` / `explain_spec` / `log_compile`
(src/palladium/diagnostics.py:21-82): `explain()` returns one of these, and
setting PALLADIUM_EXPLAIN=1 prints one stderr line per newly bound kernel.
The reference's four fields keep their names and their place in `str()`;
`msl_lines` counts the lines of the CUDA source the family is compiled from
(the analogue of the emitted MSL), and the CUDA launch geometry is appended.
"""

from __future__ import annotations

import dataclasses
import os
import sys
from functools import lru_cache
from pathlib import Path

from . import _native
from .families import KernelSpec
from .math_mode import math_mode_ordinal

__all__ = ["KernelDiagnostics", "explain_spec", "log_compile"]


@dataclasses.dataclass(frozen=True)
class KernelDiagnostics:
    """How one call will execute.

    name, grid, threadgroup, msl_lines: as in the reference
    (src/palladium/diagnostics.py:21-39).  cuda_kernel .. blocks_per_sm: the
    CUDA launch the native library will perform for that grid; register,
    shared-memory and occupancy figures are -1 where no GPU is present."""

    name: str
    grid: tuple[int, ...]
    threadgroup: tuple[int, ...] | None
    msl_lines: int
    cuda_kernel: str = ""
    cuda_grid: tuple[int, ...] = ()
    cuda_block: tuple[int, ...] = ()
    items_per_thread: int = 1
    launches: int = 1
    scratch_bytes: int = 0
    regs: int = -1
    smem_bytes: int = -1
    blocks_per_sm: int = -1

    def __str__(self) -> str:
        parts = [f"palladium kernel {self.name}: grid={self.grid}"]
        if self.threadgroup is not None:
            parts.append(f"threadgroup={self.threadgroup}")
        parts.append(f"msl_lines={self.msl_lines}")
        if self.cuda_kernel:
            parts.append(f"cuda={self.cuda_kernel}<<<{self.cuda_grid}, {self.cuda_block}>>>")
            parts.append(f"items_per_thread={self.items_per_thread}")
            parts.append(f"launches={self.launches}")
            if self.regs >= 0:
                parts.append(f"regs={self.regs} smem={self.smem_bytes} blocks_per_sm={self.blocks_per_sm}")
        return " ".join(parts)


@lru_cache(maxsize=1)
def _source_lines() -> int:
    src = Path(__file__).resolve().parent / "csrc" / "pd_kernels.cu"
    try:
        return len(src.read_text().splitlines())
    except OSError:
        return 0


def _normalise_threadgroup(threadgroup) -> tuple[int, ...] | None:
    if threadgroup is None:
        return None
    if isinstance(threadgroup, int):
        return (threadgroup,)
    return tuple(int(t) for t in threadgroup)


def explain_spec(spec: KernelSpec, threadgroup=None, math_mode="fast") -> KernelDiagnostics:
    """Diagnostics for a validated call: asks the native library for the launch
    plan; dispatches nothing.  (A run-time right-hand side is compiled, and
    cached, if a GPU is present: its register count is part of the report.)"""
    tg = _normalise_threadgroup(threadgroup)
    if spec.family.name == "custom_ode":
        lines = len(spec.family.constants["rhs"].splitlines())
    elif spec.family.name == "source":
        lines = len(spec.family.constants["source"].splitlines())
    else:
        lines = _source_lines()
    info = _native.explain(spec.family.family_id, spec.params, math_mode_ordinal(math_mode), spec.grid, tg)
    return KernelDiagnostics(
        name=spec.name,
        grid=tuple(int(g) for g in spec.grid),
        threadgroup=tg,
        msl_lines=lines,
        cuda_kernel=info.kernel_name.decode(),
        cuda_grid=tuple(int(v) for v in info.cuda_grid),
        cuda_block=tuple(int(v) for v in info.cuda_block),
        items_per_thread=int(info.items_per_thread),
        launches=int(info.launches),
        scratch_bytes=int(info.scratch_bytes),
        regs=int(info.regs_per_thread),
        smem_bytes=int(info.static_smem_bytes),
        blocks_per_sm=int(info.blocks_per_sm),
    )


def _explain_enabled() -> bool:
    return os.environ.get("PALLADIUM_EXPLAIN", "") not in ("", "0")


def log_compile(spec: KernelSpec, threadgroup=None, math_mode="fast") -> None:
    """One stderr line per newly bound kernel when PALLADIUM_EXPLAIN is set;
    called on the cache-miss path only, so cached shapes stay silent."""
    if _explain_enabled():
        print(explain_spec(spec, threadgroup, math_mode), file=sys.stderr)
