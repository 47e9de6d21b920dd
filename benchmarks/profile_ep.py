#!/usr/bin/env python
"""Small single-GPU instance of MoE dispatch + combine for profiler captures.

Sized so that a capture ends by itself: one PE, a 2 GiB heap, 8192 tokens of hidden 7168 (inputs and
outputs together exceed the 126 MB L2, so DRAM counters mean something), a handful of launches.

    python benchmarks/profile_ep.py --steps 3
    ncu --set full --clock-control none -k regex:ep_dispatch -c 2 -o bench_out/ep_dispatch \
        python benchmarks/profile_ep.py --steps 3
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.ops import moe  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    shm.init(heap_size=2 << 30, device=0)
    T, H, E, K = args.tokens, args.hidden, 256, 8
    d = moe.EpDispatcher(E, K, H, T)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    idx, w = moe.make_routing(T, E, K, 1, "cuda")
    y = d.result_buffer()
    y.normal_()
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    for i in range(args.steps):
        start.record()
        d.dispatch(x, idx, w)
        d.combine(y, idx, w, T, weighted=True, out=out)
        end.record()
        torch.cuda.synchronize()
        print(f"step {i}: {start.elapsed_time(end) * 1e3:.1f} us", d.phase_times_us())
    err = shm.get_error()
    assert err["count"] == 0, err
    shm.finalize()


if __name__ == "__main__":
    main()
