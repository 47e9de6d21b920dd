#!/usr/bin/env python
"""Collective and RMA micro-benchmarks on the symmetric heap, with NCCL on the same GPUs as baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29544 benchmarks/coll_bench.py --out bench_out/coll_n8.json

    ... benchmarks/coll_bench.py --teams 2,4,8 --dtypes bfloat16,float32 --size-step 2 --only allreduce,copies

For every team size (the first k PEs; the world team by default), element type and message size: device time (CUDA
events, maximum over the team's members, L2 not flushed because the payloads above 128 MiB exceed it and the small
ones are latency-bound) of

* allreduce: flag-in-word (up to 2 KiB), one-shot, two-shot, NVLS (world team, when available) kernels of this
  library, and ``ncclAllReduce``; bus bandwidth = 2 (n-1)/n * bytes / time; one result per run is checked against
  an fp64 sum of the members' inputs;
* fcollect (all-gather), alltoall, broadcast: this library's kernels, with and without their entry barrier, and
  the NCCL equivalents;
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
    ap.add_argument("--dtypes", default="bfloat16", help="comma list of: bfloat16, float32")
    ap.add_argument("--teams", default="", help="comma list of team sizes (first k PEs); default: the world team only")
    ap.add_argument("--size-step", type=int, default=1, help="message sizes grow by 2^step")
    ap.add_argument("--only", default="allreduce,copies,rma", help="comma list of: allreduce, copies, rma")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29544")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    shm.init(heap_size=8 << 30, device=local)
    k = _native.load_test_kernels()
    only = set(args.only.split(","))
    team_sizes = [int(t) for t in args.teams.split(",") if t] or [world]
    results = {"n_gpus": world, "nvls": shm.nvls_available(), "runs": [], "rma": []}
    src8 = shm.zeros(args.max_bytes, torch.uint8)
    dst8 = shm.zeros(args.max_bytes, torch.uint8)
    nccl8 = torch.empty(args.max_bytes, dtype=torch.uint8, device="cuda")
    out8 = torch.empty(args.max_bytes, dtype=torch.uint8, device="cuda")
    for tsize in team_sizes:
        if tsize > world or tsize < 2:
            continue
        # Every PE takes part in the split and in new_group; only members run the timed loops.
        team = shm.team_world() if tsize == world else shm.team_world().split_strided(0, 1, tsize)
        group = dist.group.WORLD if tsize == world else dist.new_group(list(range(tsize)))
        member = rank < tsize
        for dtype_name in args.dtypes.split(","):
            dtype = getattr(torch, dtype_name)
            esz = torch.empty((), dtype=dtype).element_size()
            src, dst = src8.view(dtype), dst8.view(dtype)
            nccl_buf, out_nccl = nccl8.view(dtype), out8.view(dtype)
            src.normal_()
            nccl_buf.normal_()
            torch.cuda.synchronize()
            shm.barrier_all()
            run = {"team_size": tsize, "dtype": dtype_name, "allreduce": [], "fcollect": [], "alltoall": [],
                   "broadcast": []}

            def timed_team(fn, iters, warmup=3):
                """Device time in microseconds, maximum over the team's members."""
                us = torch.zeros(1, device="cuda")
                if member:
                    for _ in range(warmup):
                        fn()
                    torch.cuda.synchronize()
                    dist.barrier(group=group)
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    for _ in range(iters):
                        fn()
                    end.record()
                    torch.cuda.synchronize()
                    us[0] = start.elapsed_time(end) * 1e3 / iters
                    dist.all_reduce(us, op=dist.ReduceOp.MAX, group=group)
                return float(us.item())

            # One allreduce checked against an fp64 sum of every member's input (gathered over NCCL).
            if member:
                n_chk = 4096
                coll.allreduce_async(dst[:n_chk], src[:n_chk], shm.OP_SUM, team=team)
                parts = [torch.empty(n_chk, dtype=dtype, device="cuda") for _ in range(tsize)]
                dist.all_gather(parts, src[:n_chk].clone(), group=group)
                want = sum(p.double() for p in parts)
                tol = 1e-5 if dtype == torch.float32 else 3e-2
                run["allreduce_max_err_vs_fp64"] = float((dst[:n_chk].double() - want).abs().max())
                run["verified"] = bool(run["allreduce_max_err_vs_fp64"] <= tol * max(1.0, float(want.abs().max())))
            sizes = [1 << p for p in range(9, 40, args.size_step) if (1 << p) <= args.max_bytes]
            busf = 2 * (tsize - 1) / tsize
            for nbytes in (sizes if "allreduce" in only else []):
                n = nbytes // esz
                iters = 50 if nbytes <= (1 << 20) else (10 if nbytes <= (64 << 20) else 4)
                row = {"bytes": nbytes, "elements": n}
                algos = {"one_shot": shm.ALLREDUCE_ONE_SHOT, "two_shot": shm.ALLREDUCE_TWO_SHOT,
                         "auto": shm.ALLREDUCE_AUTO}
                if nbytes <= 2048:
                    algos["ll"] = shm.ALLREDUCE_LL
                if member and team.has_nvls():      # the world team's mapping, or a split team's own object
                    algos["nvls"] = shm.ALLREDUCE_NVLS
                for name, algo in algos.items():
                    if name == "one_shot" and nbytes > (8 << 20):
                        continue
                    us = timed_team(lambda: coll.allreduce_async(dst[:n], src[:n], shm.OP_SUM, team=team, algo=algo), iters)
                    row[name + "_us"] = us
                    row[name + "_busbw_gbs"] = busf * nbytes / us / 1e3 if us else None
                us = timed_team(lambda: dist.all_reduce(nccl_buf[:n], group=group), iters)
                row["nccl_us"], row["nccl_busbw_gbs"] = us, busf * nbytes / us / 1e3 if us else None
                run["allreduce"].append(row)
                if rank == 0:
                    print("allreduce", tsize, dtype_name, {kk: (round(v, 1) if isinstance(v, float) else v) for kk, v in row.items()}, flush=True)
            # all-gather / all-to-all / broadcast: per-peer payload 4 KiB ... 128 MiB (bounded by the buffers).
            # Ours is timed twice: without the entry barrier (the caller knows the destinations are free) and with
            # it (what NCCL's own synchronisation corresponds to).
            per_peer = [1 << p for p in range(12, 28, args.size_step) if (1 << p) * tsize <= args.max_bytes]
            for nbytes in (per_peer if "copies" in only else []):
                n = nbytes // esz
                iters = 30 if nbytes <= (1 << 20) else 6
                for name, ours, theirs in (
                    ("fcollect", lambda ps: coll.fcollect_async(dst[:n * tsize], src[:n], team=team, pre_sync=ps),
                     lambda: dist.all_gather_into_tensor(out_nccl[:n * tsize], nccl_buf[:n], group=group)),
                    ("alltoall", lambda ps: coll.alltoall_async(dst[:n * tsize], src[:n * tsize], team=team, pre_sync=ps),
                     lambda: dist.all_to_all_single(out_nccl[:n * tsize], nccl_buf[:n * tsize], group=group)),
                    ("broadcast", lambda ps: coll.broadcast_async(dst[:n], src[:n], 0, team=team, pre_sync=ps),
                     lambda: dist.broadcast(nccl_buf[:n], 0, group=group)),
                ):
                    us = timed_team(lambda: ours(False), iters)
                    us_sync = timed_team(lambda: ours(True), iters)
                    us_nccl = timed_team(theirs, iters)
                    moved = nbytes * (tsize - 1) if name != "broadcast" else nbytes
                    row = {"bytes_per_peer": nbytes, "us": us, "gbs": moved / us / 1e3 if us else None,
                           "us_pre_sync": us_sync, "gbs_pre_sync": moved / us_sync / 1e3 if us_sync else None,
                           "nccl_us": us_nccl, "nccl_gbs": moved / us_nccl / 1e3 if us_nccl else None}
                    run[name].append(row)
                    if rank == 0:
                        print(name, tsize, dtype_name, {kk: (round(v, 1) if isinstance(v, float) else v) for kk, v in row.items()}, flush=True)
            results["runs"].append(run)
        torch.cuda.synchronize()
        shm.barrier_all()
        if tsize != world and team.valid:
            team.destroy()
    src, dst = src8, dst8
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
