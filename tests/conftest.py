"""pytest configuration: the ``gpu`` marker and shared helpers.

Tests marked ``gpu`` need a B200 and call the CUDA library through its C-ABI; everything else runs
on CPU (oracle against the golden fixtures, host logic, symbol export checks, gloo ranks).
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(GOLDEN / f"{name}.npz")

    return load
