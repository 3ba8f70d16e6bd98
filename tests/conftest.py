import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def _have_gpu() -> bool:
    try:
        from vkml_b200 import _abi
        import ctypes
        n = ctypes.c_int(0)
        return _abi.load().b200_device_count(ctypes.byref(n)) == 0 and n.value > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def backend():
    """One CUDA backend for the whole session (GPU tests only)."""
    import vkml_b200
    b = vkml_b200.Backend(0)
    yield b
    b.synchronize()


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this environment")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
