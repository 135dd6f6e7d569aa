import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")
    config.addinivalue_line("markers", "perf: performance floors on a B200; selected only with `-m perf`")


def pytest_collection_modifyitems(config, items):
    # the performance tier only runs when it is asked for by name (timing tests do not belong in a correctness run)
    # RUSTRAL_RUN_GPU_PERF=1 selects the tier as well (the switch of the reference's tests/performance/gpu.rs)
    perf_selected = "perf" in (config.getoption("-m") or "") or os.environ.get("RUSTRAL_RUN_GPU_PERF") == "1"
    skip_perf = pytest.mark.skip(reason="performance tier: select it with `-m perf` or RUSTRAL_RUN_GPU_PERF=1 on a B200")
    skip = pytest.mark.skip(reason="no CUDA device")
    have_gpu = torch.cuda.is_available()
    if not have_gpu and os.environ.get("RUSTRAL_REQUIRE_GPU") == "1":
        # fail fast instead of skipping every GPU test (crates/wgpu-backend/tests/correctness.rs:8-22)
        raise pytest.UsageError("RUSTRAL_REQUIRE_GPU=1 but no CUDA device is available")
    for item in items:
        if "perf" in item.keywords and not (perf_selected and have_gpu):
            item.add_marker(skip_perf)
        elif not have_gpu and ("gpu" in item.keywords or "multigpu" in item.keywords):
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
