import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "triton-kernels_b200")
for p in (PKG, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_error_check(request):
    """After every GPU test, fail if a kernel recorded a device-side error
    (bounded wait expired, block-table entry out of range)."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from kernels import _native

        torch.cuda.synchronize()
        _native.check_device_errors()
