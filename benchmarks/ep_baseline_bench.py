#!/usr/bin/env python
"""The headline dispatch + combine workload of ``bench.py`` on the library baseline: ``torch.distributed``
all-to-all over NCCL (``rocshmem_b200.baselines.ep.NcclEpDispatcher``), same shapes, same routing, same timing
rules (CUDA events on the launching stream, L2 flushed between steps, maximum over ranks).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/ep_baseline_bench.py

Prints one JSON line on rank 0; ``--out`` also writes it to a file. Put it next to the line of
``bench.py --gpus N`` to compare.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rocshmem_b200.baselines.ep import NcclEpDispatcher  # noqa: E402
from rocshmem_b200.ops import moe  # noqa: E402

EXPERTS, TOPK, HIDDEN, TOKENS = 256, 8, 7168, 4096


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=TOKENS)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    T = args.tokens
    d = NcclEpDispatcher(EXPERTS, TOPK, HIDDEN)
    g = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(T, HIDDEN, generator=g).to(torch.bfloat16).to(dev)
    idx_cpu, w_cpu = moe.make_routing(T, EXPERTS, TOPK, 99 + rank)
    idx, w = idx_cpu.to(dev), w_cpu.to(dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    res = d.dispatch(x, idx, w)
    y = moe.ref_dequantize_1x128(res.recv_x, res.recv_scales).to(torch.bfloat16)

    def step(events=None):
        if events:
            events[0].record()
        d.dispatch(x, idx, w)
        if events:
            events[1].record()
        d.combine(y, idx, w, T)
        if events:
            events[2].record()

    for _ in range(max(3, args.warmup)):
        flush.fill_(1)
        step()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    before = d.collectives
    for i in range(args.steps):
        flush.fill_(i & 0xff)
        step(ev[i])
    torch.cuda.synchronize()
    dist.barrier()
    disp = sum(e[0].elapsed_time(e[1]) for e in ev)
    comb = sum(e[1].elapsed_time(e[2]) for e in ev)
    t = torch.tensor([disp + comb, disp, comb], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, disp_ms, comb_ms = t.tolist()
    if rank == 0:
        ms = total_ms / args.steps
        line = {"metric": "ep_dispatch_combine_tokens_per_s", "value": world * T / (ms * 1e-3), "unit": "tokens/s",
                "impl": "nccl all_to_all_single baseline", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms, "dispatch_us": disp_ms / args.steps * 1e3, "combine_us": comb_ms / args.steps * 1e3,
                "collectives_per_step": (d.collectives - before) / args.steps,
                "config": {"experts": EXPERTS, "top_k": TOPK, "hidden": HIDDEN, "tokens_per_rank": T,
                           "dispatch": "fp8 e4m3 + fp32 scale per 128 (torch kernels)", "combine": "bf16, weighted sum",
                           "l2": "flushed between steps (512 MiB write)"}}
        print(json.dumps(line))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(line, f)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
