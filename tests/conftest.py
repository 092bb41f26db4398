import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# The CPU suite runs tiny models: intra-op parallelism over every core costs more in thread hand-offs than it saves, and
# the multi-process tests share the cores between ranks.
if not torch.cuda.is_available():
    torch.set_num_threads(min(4, os.cpu_count() or 1))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    if torch.cuda.is_available():
        from stkernel_b200.ops import _lib
        if _lib._status:
            torch.cuda.synchronize()
            _lib.check_status()
