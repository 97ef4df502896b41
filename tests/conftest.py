"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; everything
else runs on the CPU (oracle against the golden vectors, host logic, symbol
checks of the C-ABI library, gloo multi-process sharding logic)."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "helpers_golden.npz")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    from cwm_b200 import _lib, build

    build.build()
    return _lib.load()
