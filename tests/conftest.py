import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "ml-autofocusformer_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def lib():
    """libclusten_b200.so, built on demand (nvcc cross-compiles without a GPU)."""
    import build as _build  # ml-autofocusformer_b200/build.py
    _build.build()
    from clusten import _lib
    return _lib.load()
