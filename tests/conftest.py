import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multi_gpu: needs at least two CUDA devices")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        ngpu = torch.cuda.device_count()
        skip_multi = pytest.mark.skip(reason="needs >= 2 GPUs")
        for item in items:
            if "multi_gpu" in item.keywords and ngpu < 2:
                item.add_marker(skip_multi)
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multi_gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _fresh_parallel_state():
    yield
    try:
        from omni_npu_b200.parallel import state
        if state.model_parallel_is_initialized() and state.get_world_group().world_size == 1:
            state.destroy_model_parallel()
    except Exception:
        pass


@pytest.fixture(autouse=True)
def _no_kernel_gave_up(request):
    """Every GPU test ends with the device status word at rest: a kernel whose bounded wait
    expired (or that rejected its arguments) fails the test that launched it, not a later one."""
    yield
    if "gpu" not in request.keywords:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from omni_npu_b200 import ops
    if getattr(ops, "_states", None):
        ops.check_status()
