"""Shared fixtures.  ``gpu`` marks tests that need a CUDA device and the built
sm_100a library; everything else must pass on a GPU-less machine."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Vectors recorded from the reference's own CPU code (tests/golden/make_golden.py)."""
    return dict(np.load(ROOT / "tests" / "golden" / "reference_vectors.npz"))
