"""Test configuration: the ``gpu`` marker and shared fixtures."""

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
    """Golden vectors produced by the reference (tests/golden/make_golden.py)."""
    merged = {}
    for name in ("packed_golden.npz", "legacy_formats_golden.npz"):
        with np.load(ROOT / "tests" / "golden" / name) as data:
            merged.update({key: data[key] for key in data.files})
    return merged


@pytest.fixture(scope="session")
def cuda():
    """torch with a CUDA device, or skip."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch
