"""Shared fixtures.  GPU tests carry the `gpu` marker; everything else runs on a
CPU-only box.  The oracle (tests' checker) is built on demand; the CUDA library
is built on demand when nvcc is present."""

import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    from oracle import build as oracle_build
    from palladium_b200 import build as lib_build

    oracle_build.build_oracle()
    oracle_build.build_reference()
    if lib_build.is_stale():
        lib_build.build()


@pytest.fixture
def rng():
    # the reference's fixture: tests/conftest.py:21-23
    return np.random.default_rng(seed=17)


@pytest.fixture(scope="session")
def has_gpu():
    import torch

    return torch.cuda.is_available()


@pytest.fixture(autouse=True)
def _gpu_guard(request):
    """A test marked gpu must never pass silently without a device."""
    if request.node.get_closest_marker("gpu"):
        import torch

        if not torch.cuda.is_available():
            pytest.fail("test is marked gpu but no CUDA device is visible")
    yield


@pytest.fixture(scope="session")
def interpret_provider():
    """Registers the CPU oracle as the `.interpret` provider for the session."""
    import palladium_b200 as pd
    from tests import oracle_provider

    previous = pd.register_interpret_provider(oracle_provider.interpret)
    yield oracle_provider.interpret
    pd.register_interpret_provider(previous)
