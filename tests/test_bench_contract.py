"""The benchmark entry point: the reference arm's answer (no GPU needed) and, on a GPU, the single-line report of
a short run."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable_and_exits_zero():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-1000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


@pytest.mark.gpu
def test_a_short_run_prints_one_json_line_with_the_contract_keys():
    """A real (small) run on one GPU: the last line of stdout is the report."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "1", "--steps", "2", "--warmup", "3",
                          "--tokens", "256", "--repeats", "2"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-2000:])
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "verified", "baseline"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 3 and line["verified"] is True
    assert line["value"] > 0 and line["gpu_launches"] == 2 * 2 * 2          # steps x pairs x (dispatch + combine)
    assert line["e2e"]["h2d_bytes_per_step"] == 256 * 7168 * 2 + 2 * 256 * 8 * 4 and line["e2e"]["value"] > 0
    ll = line["extra"]["low_latency_128_tokens"]
    assert ll is not None and "error" not in ll and ll["verified"] is True and ll["dispatch_us"] > 0, ll
    assert line["baseline"]["value"] > 0 and abs(line["vs_baseline"] - line["value"] / line["baseline"]["value"]) < 1e-6
