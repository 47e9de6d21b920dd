"""Roofline arithmetic shared by the benchmarks: measured peaks of this pool and achieved fractions."""
from __future__ import annotations

import json
import os
from typing import Optional

NVLINK_MEASURED_GBS = 770.0      # peer copy, per direction and GPU, measured on this pool
NVLINK_NOMINAL_GBS = 900.0
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks(root: Optional[str] = None) -> dict:
    """The pool's measured peaks (``MEASURED_PEAKS.json`` at the repository root) or the documented fallback;
    the returned dict carries ``"source": "measured" | "fallback"``."""
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        out = {k: float(p[k]) for k in FALLBACK}
        out["source"] = "measured"
        return out
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK, source="fallback")


def memory_fraction(bytes_moved: float, seconds: float, peaks: Optional[dict] = None) -> float:
    """Achieved bytes per second as a fraction of the measured copy bandwidth."""
    peaks = peaks or measured_peaks()
    return bytes_moved / seconds / 1e9 / peaks["hbm_gbs"]


def compute_fraction(flops: float, seconds: float, sustained: bool = False, peaks: Optional[dict] = None) -> float:
    """Achieved FLOP/s as a fraction of the measured cuBLAS bf16 throughput (burst or sustained)."""
    peaks = peaks or measured_peaks()
    return flops / seconds / 1e12 / peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]


def fused_roofline_seconds(flops: float, nvlink_bytes_per_direction: float, sustained: bool = True,
                           peaks: Optional[dict] = None) -> float:
    """Target time of a fused compute + collective kernel: the slower of the math at the measured GEMM peak
    and the bytes that must cross NVLink at the measured link bandwidth."""
    peaks = peaks or measured_peaks()
    tf = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    return max(flops / (tf * 1e12), nvlink_bytes_per_direction / (NVLINK_MEASURED_GBS * 1e9))
