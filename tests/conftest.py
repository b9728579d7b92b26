import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library; building it needs nvcc but no GPU."""
    from batchlas_b200 import build as _build
    _build.build()
    from batchlas_b200 import _lib
    return _lib.load()
