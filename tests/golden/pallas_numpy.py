"""NumPy stand-ins for the handful of `jax.numpy`, `jax.lax`, `jax.random` and
`pl` names the reference's example kernels use, so that the *reference's own
kernel functions* can be executed here, where JAX is not installed, to produce
known-answer fixtures (tests/golden/make_golden.py).  TEST INFRASTRUCTURE ONLY.

The kernels are written for one program instance per trajectory with blocks of
one element; every operation in them is elementwise, so running the body once
on whole (N,) arrays performs, per element, exactly the operations one program
instance performs.  What has to be reproduced is JAX's typing:

* float32 arrays stay float32 when combined with Python scalars (NumPy >= 2
  does the same), and a Python scalar handed to a jnp function alone becomes
  float32 (`jnp.sqrt(dt)`), as does `jnp.where(c, 1.0, 0.0)`;
* `x ** 2` is a multiplication; `x ** c` for a float c is the float32 `pow`.

pow / exp / log / cos / sqrt go through the C library (oracle.libm_f32) so that
the results can be compared bit for bit with the C oracle, which calls the
same functions; NumPy's own float32 loops for them round differently.
RNG calls use the restatement whose Threefry block is pinned separately
(tests/golden/threefry_reference.npz).
"""

from __future__ import annotations

import ast
import math
from pathlib import Path

import numpy as np

import oracle
from oracle import oracle_np


class F32(np.ndarray):
    """float32 array whose `**` follows JAX: integer 2 -> x*x, float -> powf."""

    def __pow__(self, exponent):
        if isinstance(exponent, int) and exponent == 2:
            return self * self
        return oracle.libm_f32("pow", np.asarray(self), np.float32(exponent)).view(F32)


def f32(a) -> F32:
    return np.ascontiguousarray(a, np.float32).view(F32)


def _weak(x):
    """A lone Python scalar takes JAX's default float type."""
    return np.float32(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else x


def _wrap(a):
    a = np.asarray(a)
    return a.view(F32) if a.dtype == np.float32 else a


class _Jnp:
    pi = math.pi
    float32 = np.float32

    @staticmethod
    def where(c, a, b):
        if isinstance(a, float) or isinstance(b, float):
            a, b = _weak(a), _weak(b)
        return _wrap(np.where(c, a, b))

    @staticmethod
    def minimum(a, b):
        return _wrap(np.minimum(a, b))

    @staticmethod
    def maximum(a, b):
        return _wrap(np.maximum(a, b))

    @staticmethod
    def clip(a, lo, hi):
        return _wrap(np.minimum(np.maximum(a, lo), hi))

    @staticmethod
    def abs(a):
        return _wrap(np.abs(a))

    @staticmethod
    def zeros_like(a):
        return f32(np.zeros_like(a))

    @staticmethod
    def ones_like(a):
        return f32(np.ones_like(a))

    @staticmethod
    def full_like(a, value):
        return f32(np.full_like(a, value))

    @staticmethod
    def sqrt(a):
        return _wrap(oracle.libm_f32("sqrt", _weak(a)))

    @staticmethod
    def log(a):
        return _wrap(oracle.libm_f32("log", _weak(a)))

    @staticmethod
    def cos(a):
        return _wrap(oracle.libm_f32("cos", _weak(a)))

    @staticmethod
    def exp(a):
        return _wrap(oracle.libm_f32("exp", _weak(a)))


class _Lax:
    @staticmethod
    def fori_loop(lo, hi, body, init):
        carry = init
        for i in range(lo, hi):
            carry = body(i, carry)
        return carry


class _Key:
    """(..., 2) uint32 key data; one key per program instance once folded with the thread id."""

    def __init__(self, data):
        self.data = np.asarray(data, np.uint32)


class _Random:
    @staticmethod
    def wrap_key_data(data, impl=None):
        assert impl in (None, "threefry2x32")
        return _Key(np.asarray(data, np.uint32).reshape(2))

    @staticmethod
    def fold_in(key: _Key, data):
        k = key.data
        d = np.asarray(data).astype(np.uint32)
        a, b = oracle_np.threefry2x32(k[..., 0], k[..., 1], np.uint32(0), d)
        return _Key(np.stack(np.broadcast_arrays(a, b), axis=-1))

    @staticmethod
    def uniform(key: _Key, shape=()):
        assert shape == ()
        k = key.data
        a, b = oracle_np.threefry2x32(k[..., 0], k[..., 1], np.uint32(0), np.uint32(0))
        bits = a ^ b
        return f32(((bits >> np.uint32(9)) | np.uint32(0x3F800000)).view(np.float32) - np.float32(1.0))


class _Jax:
    lax = _Lax
    random = _Random


class _Pl:
    """`pl.program_id(axis)` as an index array broadcast over the grid."""

    def __init__(self, grid):
        self.grid = tuple(grid)

    def program_id(self, axis):
        shape = [1] * len(self.grid)
        shape[axis] = self.grid[axis]
        return np.arange(self.grid[axis]).reshape(shape)


class Ref:
    """A whole-array stand-in for a Pallas ref: `ref[...]` reads the array,
    `ref[i, j]` indexes with (broadcast) program ids, assignment stores."""

    def __init__(self, array):
        self.array = array

    def __getitem__(self, index):
        if index is Ellipsis:
            return self.array
        return _wrap(self.array[index])

    def __setitem__(self, index, value):
        if index is Ellipsis or index == 0:
            self.array[...] = np.broadcast_to(value, self.array.shape) if np.ndim(value) else value
        else:
            self.array[index] = value


def extract_function(path: Path, name: str, outer: str | None = None) -> ast.FunctionDef:
    """The FunctionDef `name` of the module at `path`, or of its function `outer`."""
    tree = ast.parse(path.read_text())
    body = tree.body
    if outer is not None:
        body = next(n for n in body if isinstance(n, ast.FunctionDef) and n.name == outer).body
    return next(n for n in body if isinstance(n, ast.FunctionDef) and n.name == name)


def load_kernel(path: Path, name: str, grid, constants: dict, outer: str | None = None):
    """Compile one kernel function of a reference example against the stand-ins."""
    node = extract_function(path, name, outer)
    namespace = {"jnp": _Jnp, "jax": _Jax, "pl": _Pl(grid), "np": np}
    namespace.update(constants)
    exec(compile(ast.Module(body=[node], type_ignores=[]), str(path), "exec"), namespace)
    return namespace[name]
