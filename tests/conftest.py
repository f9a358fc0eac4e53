import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(autouse=True)
def _check_device_status(request):
    """After every GPU test, fail if a kernel recorded a bounded-wait timeout."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from torsh_b200 import _native as nv
            torch.cuda.synchronize()
            nv.check_status()
