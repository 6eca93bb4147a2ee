import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _cuda_available() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def skl():
    """The product library (built on demand), as the ctypes handle."""
    import skl_b200
    from skl_b200 import _build

    if not os.path.exists(skl_b200.LIB_PATH):
        _build.build()
    return skl_b200.lib()


@pytest.fixture(scope="session")
def oracle():
    from oracle import pyoracle

    pyoracle.port()
    return pyoracle
