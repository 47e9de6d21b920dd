"""Test configuration. Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs on a
machine without one (host-memory backend, multi-process over the loopback interface)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without a GPU is skipped rather than failed when it is selected anyway.
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


@pytest.fixture
def fresh_runtime():
    """Guarantees that no runtime is left initialised by the test."""
    import rocshmem_b200 as shm
    if shm.is_initialized():
        shm.finalize()
    yield shm
    if shm.is_initialized():
        shm.finalize()
