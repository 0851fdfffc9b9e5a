import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _fresh_device_status(request):
    """GPU tests start without device-side findings left by an earlier test (some tests provoke them on
    purpose: an invalid group list, an expired wait)."""
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            import ascend_kernel_b200 as ak
            from ascend_kernel_b200 import cinfer_ascendc

            ak.last_status(clear=True)
            cinfer_ascendc.last_status(True)
    yield
