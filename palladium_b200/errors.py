"""Exception hierarchy, the same five classes and base-class pairings as the
reference (src/palladium/errors.py:19-44) so that `except` clauses written
against it keep working: everything derives from PalladiumError; TraceError is
also a ValueError, UnsupportedPrimitiveError a NotImplementedError and
DispatchError a TypeError."""

from __future__ import annotations

__all__ = [
    "DispatchError",
    "EmitError",
    "PalladiumError",
    "TraceError",
    "UnsupportedPrimitiveError",
]


class PalladiumError(Exception):
    """Base class for every error this package raises."""


class TraceError(PalladiumError, ValueError):
    """The call's grid / in_specs / out_specs / out_shape do not describe a
    launch the kernel family can perform (the stage at which the reference
    fails to trace a pallas_call into a KernelSpec)."""


class EmitError(PalladiumError):
    """The native library cannot provide a kernel for this request (missing or
    stale library, unsupported launch geometry)."""


class UnsupportedPrimitiveError(EmitError, NotImplementedError):
    """The kernel handed to `cuda_call` is not one of the hand-written families
    (the reference raises this for a primitive with no lowering rule; here there
    is no emitter, so an arbitrary Pallas function has no CUDA kernel)."""


class DispatchError(PalladiumError, TypeError):
    """A bound kernel was called with arguments that do not match its traced
    spec (wrong count, shape, or dtype), or no CUDA device is available."""
