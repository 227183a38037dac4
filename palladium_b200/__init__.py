"""palladium_b200: the ensemble-integrator hot path of palladium on B200.

Pipeline of the reference: trace (Pallas -> KernelSpec) -> emit (KernelSpec ->
MSL) -> bind (MSL -> callable) behind `metal_call` (src/palladium/__init__.py:1-7).
Here: trace (validate a `pallas_call`-shaped request against a hand-written
kernel family) -> bind (family -> C-ABI launch in libpalladium_cuda.so) behind
`cuda_call`, which keeps `metal_call`'s signature, `.interpret`, `.explain`,
`.pin` and `.cache`; `cuda_call_jit` mirrors `metal_call_jit`.
"""

from __future__ import annotations

from . import families, pl, workloads
from .diagnostics import KernelDiagnostics
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

from .call import CudaCallable, cuda_call, debug_msl  # noqa: E402
