"""Shared fixtures. GPU tests are marked ``gpu`` and call the CUDA library
through its C-ABI; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG = os.path.join(ROOT, "vibevoice.c_b200")
if PKG not in sys.path:
    sys.path.insert(0, PKG)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "hotpath_golden.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle
