import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) and the built libbunker_cuda.so")


@pytest.fixture(scope="session")
def bk():
    """The library initialised on cuda:0.  No fallback: a missing .so or GPU is a test error."""
    from bunker_b200 import runtime as R

    R.cu(0)
    return R
