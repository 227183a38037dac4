"""What this package raises.

The class names and their second base classes are part of the interface a user
of the reference already codes against (src/palladium/errors.py:19-44 defines the
same five): `except ValueError` still catches a bad call description, `except
TypeError` a bad argument list, `except NotImplementedError` a kernel nothing can
lower.  What each one means here, where there is no emitter:

======================  =================  ===========================================
class                   also a             raised when
======================  =================  ===========================================
PalladiumError          Exception          (root of the family)
TraceError              ValueError         grid / specs / out_shape do not describe a
                                           launch of the chosen kernel family
EmitError               --                 no kernel can be provided: the native
                                           library is missing or stale, or run-time
                                           source does not compile
UnsupportedPrimitive-   EmitError,         `cuda_call` was handed something that is not
Error                   NotImplemented-    a kernel family (an arbitrary Pallas
                        Error              function has no CUDA form here)
DispatchError           TypeError          a bound kernel got the wrong number, shape
                                           or dtype of arrays, or there is no GPU
======================  =================  ===========================================
"""

from __future__ import annotations


class PalladiumError(Exception):
    pass


class EmitError(PalladiumError):
    pass


class TraceError(PalladiumError, ValueError):
    pass


class DispatchError(PalladiumError, TypeError):
    pass


class UnsupportedPrimitiveError(EmitError, NotImplementedError):
    pass


PalladiumError.__doc__ = "Root of every exception raised by palladium_b200."
EmitError.__doc__ = ("No kernel can be provided for the request: libpalladium_cuda.so is missing or was built "
                     "for another ABI, a launch geometry is unsupported, or caller-supplied source fails to compile "
                     "(the compiler's log is the message).")
TraceError.__doc__ = ("The keywords of the call (grid, in_specs, out_specs, out_shape) or the example arrays do not "
                      "describe a launch the kernel family performs.")
DispatchError.__doc__ = ("Arrays handed to a bound kernel disagree with its traced operands in count, shape or "
                         "element type, or no CUDA device is present.")
UnsupportedPrimitiveError.__doc__ = ("The object given as `kernel` is not one of palladium_b200.families: there is "
                                     "no Pallas-to-CUDA emitter, so only the families (and run-time source) run.")

__all__ = sorted(name for name, obj in list(globals().items())
                 if isinstance(obj, type) and issubclass(obj, PalladiumError))
