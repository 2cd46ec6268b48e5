"""pytest configuration: marker registration and import paths."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _tcgen05_status_clean(request):
    """After every GPU test: no bounded wait of the tcgen05 kernels may have run out."""
    yield
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            from mlstm_kernels_b200 import _lib

            assert _lib.device_status() == 0
