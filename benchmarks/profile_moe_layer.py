#!/usr/bin/env python
"""Small single-GPU instance of the MoE feed-forward layer for profiler captures: dispatch, expert layout, gather,
grouped GEMM with SwiGLU, grouped GEMM, per-pair reduction, combine - one PE, so every kernel of the layer can be
captured on one GPU.

Sized so that a capture ends by itself: 32 local experts, 4096 tokens, hidden 7168, intermediate 2048 (the weights
alone are 2.8 GB in bf16, far beyond the 126 MB L2), a handful of launches.

    python benchmarks/profile_moe_layer.py --steps 2
    ncu --set full --clock-control none -k regex:grouped_gemm -c 2 -o bench_out/grouped_gemm \
        python benchmarks/profile_moe_layer.py --steps 2
    python benchmarks/profile_moe_layer.py --fp8 --steps 2          # block-scaled e4m3 experts

Prints the device time of every stage (CUDA events) after the warm-up step.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.models import moe_ffn  # noqa: E402
from rocshmem_b200.ops import moe  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 expert GEMMs")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    shm.init(heap_size=3 << 30, device=0)
    T, H = args.tokens, args.hidden
    layer = moe_ffn.MoEFeedForward(args.experts, args.top_k, H, args.inter, max_tokens=T, seed=1, fp8_experts=args.fp8)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    idx, w = moe.make_routing(T, args.experts, args.top_k, 1, "cuda")
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    layer(x, idx, w, out=out)                      # warm-up: module loading, first-use allocations
    torch.cuda.synchronize()
    for i in range(args.steps):
        stages = {}
        layer(x, idx, w, out=out, stage_us=stages)
        print(f"step {i}: " + ", ".join(f"{k} {v:.0f} us" for k, v in stages.items()), flush=True)
    err = shm.get_error()
    assert err["count"] == 0, shm.describe_error(err)
    layer.destroy()
    shm.finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
