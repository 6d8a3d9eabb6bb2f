"""Shared test configuration.  GPU tests are marked ``gpu``; everything else runs on a CPU-only machine."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native_library():
    """The built shared library (built on demand; a missing compiler is a hard failure, not a skip)."""
    from molt_b200 import _native
    from molt_b200.build import build

    build()
    return _native.library()


def load_golden(name: str):
    return np.load(GOLDEN / f"{name}.npz")
