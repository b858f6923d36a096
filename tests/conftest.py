import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200)")


def _has_cuda():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test: no bounded wait inside a kernel may have given up."""
    yield
    if "gpu" in request.keywords and _has_cuda():
        import torch

        from nkipy_b200 import ops

        torch.cuda.synchronize()
        assert ops.device_status(reset=True) == 0
