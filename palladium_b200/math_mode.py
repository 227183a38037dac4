"""Math modes.  The reference takes `metal_runtime.MathMode`, a StrEnum with
values "safe" / "relaxed" / "fast", and converts it to the C API's ordinals
0 / 1 / 2 in one place (src/palladium/ffi.py:35-38); both spellings are kept."""

from __future__ import annotations

import enum

__all__ = ["MathMode", "math_mode_ordinal"]


class MathMode(str, enum.Enum):
    SAFE = "safe"        # IEEE op order, no FMA contraction, IEEE div/sqrt, denormals kept
    RELAXED = "relaxed"  # FMA contraction allowed; accurate div / sqrt / libm
    FAST = "fast"        # reassociation, approximate transcendentals, flush-to-zero

    def __str__(self) -> str:  # StrEnum behaviour on every supported Python
        return self.value


_ORDINALS = {"safe": 0, "relaxed": 1, "fast": 2}


def math_mode_ordinal(mode) -> int:
    """Ordinal the native handler expects; accepts a MathMode, any enum whose
    value is one of the three strings, the string itself, or the ordinal."""
    value = mode.value if hasattr(mode, "value") else mode
    if isinstance(value, str):
        try:
            return _ORDINALS[value.lower()]
        except KeyError:
            raise ValueError(f"unknown math_mode {mode!r}: expected safe, relaxed or fast") from None
    if isinstance(value, int) and 0 <= value <= 2:
        return int(value)
    raise ValueError(f"unknown math_mode {mode!r}: expected safe, relaxed or fast")
