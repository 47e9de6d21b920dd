#!/usr/bin/env python
"""Collective and RMA micro-benchmarks on the symmetric heap, with NCCL on the same GPUs as baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29544 benchmarks/coll_bench.py --out bench_out/coll_n8.json

For every message size: device time (CUDA events, maximum over ranks, L2 not flushed because the
payloads above 128 MiB exceed it and the small ones are latency-bound) of

* allreduce: one-shot, two-shot, NVLS (when available) kernels of this library, and ``ncclAllReduce``;
  bus bandwidth = 2 (n-1)/n * bytes / time;
* fcollect (all-gather), alltoall, broadcast: this library's push kernels and the NCCL equivalents;
* put / get: one PE moving a buffer to / from its neighbour with the block-scope device API.

The reference's harness prints the same quantities per size (latency in us, bandwidth), see
``tests/functional_tests/tester.cpp:488-531``; it ships no numbers.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200 import _native  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402


def timed(fn, iters, warmup=3):
    """Median-free simple average over `iters` launches, device time in microseconds (max over ranks)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    us = torch.tensor([start.elapsed_time(end) * 1e3 / iters], device="cuda")
    dist.all_reduce(us, op=dist.ReduceOp.MAX)
    return float(us.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bench_out/coll_bench.json")
    ap.add_argument("--max-bytes", type=int, default=512 << 20)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--only", default="allreduce,copies,rma", help="comma list of: allreduce, copies, rma")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    shm.init(heap_size=8 << 30, device=local)
    k = _native.load_test_kernels()
    dtype = getattr(torch, args.dtype)
    esz = torch.empty((), dtype=dtype).element_size()
    results = {"n_gpus": world, "dtype": args.dtype, "nvls": shm.nvls_available(), "allreduce": [], "fcollect": [],
               "alltoall": [], "broadcast": [], "rma": []}
    max_elems = args.max_bytes // esz
    src = shm.zeros(max_elems, dtype)
    dst = shm.zeros(max_elems, dtype)
    src.normal_()
    nccl_buf = torch.empty(max_elems, dtype=dtype, device="cuda").normal_()
    torch.cuda.synchronize()
    shm.barrier_all()
    sizes = [1 << p for p in range(9, 40) if (1 << p) <= args.max_bytes]  # 512 B ... max
    busf = 2 * (world - 1) / world if world > 1 else 1.0
    only = set(args.only.split(","))
    for nbytes in (sizes if "allreduce" in only else []):
        n = nbytes // esz
        iters = 50 if nbytes <= (1 << 20) else (10 if nbytes <= (64 << 20) else 4)
        row = {"bytes": nbytes}
        algos = {"one_shot": shm.ALLREDUCE_ONE_SHOT, "two_shot": shm.ALLREDUCE_TWO_SHOT, "auto": shm.ALLREDUCE_AUTO}
        if shm.nvls_available():
            algos["nvls"] = shm.ALLREDUCE_NVLS
        for name, algo in algos.items():
            if name == "one_shot" and nbytes > (8 << 20):
                continue
            us = timed(lambda: coll.allreduce_async(dst[:n], src[:n], shm.OP_SUM, algo=algo), iters)
            row[name + "_us"] = us
            row[name + "_busbw_gbs"] = busf * nbytes / us / 1e3
        us = timed(lambda: dist.all_reduce(nccl_buf[:n]), iters)
        row["nccl_us"], row["nccl_busbw_gbs"] = us, busf * nbytes / us / 1e3
        results["allreduce"].append(row)
        if rank == 0:
            print("allreduce", {kk: (round(v, 1) if isinstance(v, float) else v) for kk, v in row.items()}, flush=True)
    # all-gather / all-to-all / broadcast: per-peer payload 4 KiB ... 128 MiB (bounded by the buffers)
    per_peer = [1 << p for p in range(12, 28) if (1 << p) * world <= args.max_bytes]
    out_nccl = torch.empty(max_elems, dtype=dtype, device="cuda")
    for nbytes in (per_peer if "copies" in only else []):
        n = nbytes // esz
        iters = 30 if nbytes <= (1 << 20) else 6
        for name, ours, theirs in (
            ("fcollect", lambda: coll.fcollect_async(dst[:n * world], src[:n], pre_sync=False),
             lambda: dist.all_gather_into_tensor(out_nccl[:n * world], nccl_buf[:n])),
            ("alltoall", lambda: coll.alltoall_async(dst[:n * world], src[:n * world], pre_sync=False),
             lambda: dist.all_to_all_single(out_nccl[:n * world], nccl_buf[:n * world])),
            ("broadcast", lambda: coll.broadcast_async(dst[:n], src[:n], 0, pre_sync=False),
             lambda: dist.broadcast(nccl_buf[:n], 0)),
        ):
            us, us_nccl = timed(ours, iters), timed(theirs, iters)
            moved = nbytes * (world - 1) if name != "broadcast" else nbytes
            row = {"bytes_per_peer": nbytes, "us": us, "gbs": moved / us / 1e3, "nccl_us": us_nccl,
                   "nccl_gbs": moved / us_nccl / 1e3}
            results[name].append(row)
            if rank == 0:
                print(name, {kk: (round(v, 1) if isinstance(v, float) else v) for kk, v in row.items()}, flush=True)
    # put / get from PE 0 to PE 1 with the block-scope device API (device-timed inside the kernel)
    if world >= 2 and "rma" in only:
        ns = shm.zeros(256, torch.int64)
        for nbytes in [1 << p for p in range(3, 27)]:
            for mode, name in ((0, "put_nbi_block+quiet"), (1, "get_block")):
                blocks = max(1, min(128, nbytes // 65536))
                iters = 20 if nbytes <= (1 << 20) else 4
                k.bw(mode, dst.data_ptr(), src.data_ptr(), nbytes, 1, iters, ns.data_ptr(), blocks, 512,
                     torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                shm.barrier_all()
                if rank == 0:
                    t_ns = float(ns[:blocks].max().item()) / iters
                    row = {"op": name, "bytes": nbytes, "blocks": blocks, "us": t_ns / 1e3, "gbs": nbytes / t_ns}
                    results["rma"].append(row)
                    print("rma", {kk: (round(v, 2) if isinstance(v, float) else v) for kk, v in row.items()}, flush=True)
    err = shm.get_error()
    results["errors"] = err["count"]
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    shm.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
