"""The Python examples that need no GPU, started with the launcher on the CPU shared-memory backend."""
import io
import os
import sys

import pytest

from rocshmem_b200 import launch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,world", [("data_parallel.py", 3), ("ring_attention.py", 4), ("team_allreduce.py", 5)])
def test_example_passes_on_every_rank(script, world):
    out = io.StringIO()
    rc = launch.launch([sys.executable, os.path.join(ROOT, "examples", "python", script)], world, backend="host",
                       timeout_s=200, out=out)
    text = out.getvalue()
    assert rc == 0, text[-3000:]
    assert text.count("PASS") == world and "FAIL" not in text, text[-3000:]
