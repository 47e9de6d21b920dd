"""Loads the in-tree native extension. The CUDA path must never be replaced by a silent fallback:
if the extension is missing it is built once (nvcc is part of the image); if that fails the import
fails loudly."""
from __future__ import annotations

import importlib
import os

from . import _build

_C = None
_testk = None


def load():
    """Return the ``_C`` extension module, building it on first use if it is absent."""
    global _C
    if _C is None:
        if not _build.is_built() and os.environ.get("ROCSHMEM_B200_NO_AUTOBUILD") != "1":
            _build.build(with_tests=False)
        _C = importlib.import_module("rocshmem_b200._C")
    return _C


def load_test_kernels():
    """Return the extension with the functional-test kernels (device API exercised from user code)."""
    global _testk
    load()
    if _testk is None:
        if not _build.is_built(with_tests=True):
            _build.build(with_tests=True)
        _testk = importlib.import_module("rocshmem_b200._testk")
    return _testk
