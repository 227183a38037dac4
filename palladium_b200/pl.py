"""Stand-ins for the two Pallas / JAX types a `pallas_call`-shaped signature
mentions, for environments without JAX: `BlockSpec(block_shape, index_map)` and
`ShapeDtypeStruct(shape, dtype)`.  `cuda_call` reads both by attribute
(`block_shape`, `index_map`, `shape`, `dtype`), so the real
`jax.experimental.pallas.BlockSpec` and `jax.ShapeDtypeStruct` work as well."""

from __future__ import annotations

import dataclasses
from collections.abc import Callable

import numpy as np

__all__ = ["BlockSpec", "ShapeDtypeStruct"]


@dataclasses.dataclass(frozen=True)
class BlockSpec:
    block_shape: tuple[int, ...] | None = None
    index_map: Callable[..., tuple] | None = None

    def __post_init__(self):
        if self.block_shape is not None:
            object.__setattr__(self, "block_shape", tuple(int(b) for b in self.block_shape))


@dataclasses.dataclass(frozen=True)
class ShapeDtypeStruct:
    shape: tuple[int, ...]
    dtype: np.dtype

    def __post_init__(self):
        object.__setattr__(self, "shape", tuple(int(s) for s in self.shape))
        object.__setattr__(self, "dtype", np.dtype(self.dtype))
