"""Host-side tracing helpers: NVTX ranges around library calls and a Python logger.

The reference has no trace markers (its only instrumentation is the statistics dump, src/stats.hpp, and
``DPRINTF`` under ``DEBUG``, src/util.hpp:51-71). Here ``ROCSHMEM_NVTX=1`` wraps the Python operations in
NVTX ranges so they show up by name on a timeline, and ``ROCSHMEM_DEBUG`` sets the level of the
``rocshmem_b200`` logger (0 warnings, 1 info, 2 debug).
"""
from __future__ import annotations

import contextlib
import functools
import logging
import os

log = logging.getLogger("rocshmem_b200")
if not log.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[rocshmem_b200 %(levelname)s] %(message)s"))
    log.addHandler(_h)
log.setLevel({0: logging.WARNING, 1: logging.INFO}.get(int(os.environ.get("ROCSHMEM_DEBUG", "0") or 0), logging.DEBUG))


def nvtx_enabled() -> bool:
    """True when ``ROCSHMEM_NVTX`` asks for NVTX ranges."""
    return os.environ.get("ROCSHMEM_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def trace_range(name: str):
    """NVTX range when enabled and CUDA is present, otherwise nothing."""
    if nvtx_enabled():
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
            try:
                yield
            finally:
                torch.cuda.nvtx.range_pop()
            return
    yield


def traced(name: str):
    """Decorator form of :func:`trace_range`."""
    def wrap(fn):
        @functools.wraps(fn)
        def inner(*a, **kw):
            with trace_range(name):
                return fn(*a, **kw)
        return inner
    return wrap
