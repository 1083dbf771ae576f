"""Shared fixtures.  ``gpu`` marks tests that need a CUDA device and the built
sm_100a library; everything else must pass on a GPU-less machine."""

import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
# have the decode wrappers read the device status word after every call
os.environ.setdefault("RESKV_CHECK_STATUS", "1")
for path in (str(ROOT), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Vectors recorded from the reference's own CPU code (tests/golden/make_golden.py)."""
    return dict(np.load(ROOT / "tests" / "golden" / "reference_vectors.npz"))


@pytest.fixture(scope="session")
def gpu_golden():
    """Vectors recorded from the reference's CUDA code on a B200 (tests/golden/make_golden_gpu.py)."""
    path = ROOT / "tests" / "golden" / "reference_gpu_vectors.npz"
    if not path.exists():
        pytest.skip("tests/golden/reference_gpu_vectors.npz has not been recorded")
    return dict(np.load(path))
