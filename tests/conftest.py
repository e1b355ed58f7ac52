"""Shared pytest configuration: the ``gpu`` marker and import paths."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


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
def _clean_device_status(request):
    """The device status word is sticky until read: start every GPU test with it cleared, so that a test
    that provokes a status bit (or fails before reading it) cannot fail the tests after it."""
    if "gpu" in request.keywords:
        try:
            import torch
            if torch.cuda.is_available():
                from interattn_b200 import ops
                ops.device_status()
        except Exception:
            pass
    yield
