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
    """The compiled C-ABI library; built on demand with nvcc (cross-compiles without a GPU)."""
    from trading_bot_0_b200 import _lib, build
    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def torch_node_lib(lib):
    """The libtorch autograd node library (host C++; built on demand with g++ against this image's libtorch)."""
    from trading_bot_0_b200 import build
    return build.build_torch()
