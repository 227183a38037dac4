"""The `.interpret` attribute: a CPU oracle for the same call.

In the reference `.interpret` is `pl.pallas_call(kernel, **kw, interpret=True)`
(src/palladium/__init__.py:110).  That needs JAX and the user's Pallas
function.  Resolution order here:

1. the family carries `pallas_fn` and JAX imports: exactly the reference's
   construction;
2. an interpret provider has been registered with
   `register_interpret_provider(fn)`: `fn(family, pallas_kwargs, *args)`;
3. otherwise calling `.interpret` raises PalladiumError naming both options.

The package itself ships no CPU implementation of the kernels and registers no
provider; test suites register theirs.
"""

from __future__ import annotations

import importlib.util
from collections.abc import Callable
from typing import Any

from .errors import PalladiumError

__all__ = ["interpret_callable", "register_interpret_provider"]

_provider: Callable | None = None


def register_interpret_provider(fn: Callable | None) -> Callable | None:
    """Install (or, with None, remove) the function `.interpret` falls back to
    when JAX is not installed.  Returns the previous provider."""
    global _provider
    previous, _provider = _provider, fn
    return previous


def interpret_callable(family, pallas_kwargs: dict[str, Any]) -> Callable:
    kwargs = dict(pallas_kwargs)

    def interpret(*args):
        if family.pallas_fn is not None and importlib.util.find_spec("jax") is not None:
            import jax.experimental.pallas as pl

            return pl.pallas_call(family.pallas_fn, **kwargs, interpret=True)(*args)
        if _provider is not None:
            return _provider(family, kwargs, *args)
        raise PalladiumError(
            "interpret needs either JAX plus the family's pallas_fn (the reference's "
            "pl.pallas_call(..., interpret=True)), or a provider registered with "
            "palladium_b200.register_interpret_provider; neither is available"
        )

    return interpret
