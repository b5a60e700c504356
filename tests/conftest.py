import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def vb():
    """The C-ABI library; built on demand where nvcc exists, otherwise the prebuilt .so must be there."""
    from velox_b200 import lib as L
    if not os.path.exists(L.LIB_PATH):
        from velox_b200 import build
        build.build()
    return L
