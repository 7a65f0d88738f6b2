import os
import shutil
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library is built in-tree; compile it when the checkout has none and nvcc is here."""
    from owoinfer_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH) and (shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")):
        from owoinfer_b200 import build
        build.build()
    yield
