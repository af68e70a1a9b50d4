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
