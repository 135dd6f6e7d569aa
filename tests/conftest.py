import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def cuda_status():
    """Fails the test when a kernel recorded a bounded-wait timeout or another device-side error."""
    from rustral_b200 import _native as N
    N.kernels().rb_init()
    N.read_status(clear=True)
    yield
    torch.cuda.synchronize()
    bits, where = N.read_status(clear=True)
    assert bits == 0, f"device status word set: bits={bits:#x} where={where}"
