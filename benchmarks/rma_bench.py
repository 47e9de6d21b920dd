#!/usr/bin/env python
"""Device RMA and atomic micro-benchmark, timed on the device inside the kernel.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29551 \
        benchmarks/rma_bench.py --out bench_out/rma_n2
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 ... benchmarks/rma_bench.py --all-pairs --out bench_out/rma_n8

Operations: put, get, windows of 64 put_nbi + quiet (message rate), put_signal + wait_until around a ring, int64
fetch_add and compare_swap; each at thread, warp and block scope; message sizes 8 B to 64 MiB in powers of two
(thread scope up to 1 MiB, warp scope up to 16 MiB). Payload: fp32 uniform [-1, 1) from seed 0.

Two rows per (operation, scope, size): ``groups == 1`` is one thread / warp / block moving the whole message (the
latency of a call), ``groups > 1`` spreads slices of the message over the grid (what the GPU can put on the wire).
Without ``--all-pairs`` PE 0 talks to PE 1; with it every PE talks to every other PE in turn, all at the same time,
and a row reports the slowest PE. Writes ``<out>.json`` and ``<out>.csv``. The reference prints the same columns
(size, latency, bandwidth, message rate: tests/functional_tests/tester.cpp:488-531).

``--host`` adds the latency of the host API (putmem, getmem, int64 atomic_fetch_add, barrier_all) between PE 0 and
PE 1, timed with the host clock around blocking calls.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200 import _native  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402

OPS = ["put", "get", "put_nbi_x64+quiet", "put_signal+wait_until", "fetch_add", "compare_swap"]
SCOPES = ["thread", "warp", "block"]
SCOPE_MAX = {"thread": 1 << 20, "warp": 16 << 20, "block": 64 << 20}
BLOCKS, THREADS = 128, 256


def spread_groups(scope: str, nbytes: int) -> int:
    """Groups that share a message when it is spread over the grid (a slice is at least 16 bytes / 512 bytes / 64 KiB)."""
    if scope == "thread":
        return max(1, min(BLOCKS * THREADS, nbytes // 16))
    if scope == "warp":
        return max(1, min(BLOCKS * THREADS // 32, nbytes // 512))
    return max(1, min(BLOCKS, nbytes // 65536))


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", default="bench_out/rma")
    ap.add_argument("--all-pairs", action="store_true")
    ap.add_argument("--max-bytes", type=int, default=64 << 20)
    ap.add_argument("--host", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29551")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shm.init(heap_size=1 << 30, device=local)
    k = _native.load_test_kernels()
    n_max = args.max_bytes
    src = shm.zeros(n_max // 4, torch.float32)
    dst = shm.zeros(n_max // 4, torch.float32)
    src.copy_((torch.rand(n_max // 4, generator=torch.Generator().manual_seed(0)) * 2 - 1).to(shm.device()))
    sig = shm.zeros(1, torch.int64)
    counter = shm.zeros(1, torch.int64)
    ns = shm.zeros(BLOCKS, torch.int64)
    tmax, tred = shm.zeros(1, torch.float64), shm.zeros(1, torch.float64)
    stream = torch.cuda.current_stream().cuda_stream
    rows = []
    sig_base = 0

    def run(op, scope, nbytes, groups, iters):
        nonlocal sig_base
        if groups <= 1:
            blocks = 1
        elif scope == "thread":
            blocks = (groups + THREADS - 1) // THREADS
        elif scope == "warp":
            blocks = (groups + THREADS // 32 - 1) // (THREADS // 32)
        else:
            blocks = groups
        threads = 32 if (groups <= 1 and scope != "block") else THREADS
        ns.zero_()
        counter.zero_()
        torch.cuda.synchronize()
        shm.barrier_all()
        for rep in range(2):   # the first launch warms up (module load, TLB of the peer mapping)
            k.rma_bench(OPS.index(op), SCOPES.index(scope), dst.data_ptr(), src.data_ptr(), nbytes, groups, iters,
                        int(args.all_pairs), sig.data_ptr(), counter.data_ptr(), ns.data_ptr(), sig_base, blocks, threads,
                        stream)
            torch.cuda.synchronize()
            sig_base += iters
            shm.barrier_all()
        tmax.copy_(ns[:blocks].max().double().reshape(1))
        torch.cuda.synchronize()
        coll.reduce(tred, tmax, shm.OP_MAX)
        return float(tred.cpu()[0]) / iters   # ns per round, slowest block of the slowest PE

    sizes = [1 << p for p in range(3, 27) if (1 << p) <= n_max]
    for op in OPS:
        for scope in SCOPES:
            if op in ("fetch_add", "compare_swap"):
                if scope != "thread":
                    continue
                for groups in (1, 32, BLOCKS * THREADS):
                    t = run(op, scope, 8, groups, 50)
                    rows.append({"op": op, "scope": scope, "bytes": 8, "groups": groups, "us": t / 1e3,
                                 "gbs": None, "mops": groups / t * 1e3})
                continue
            for nbytes in sizes:
                if nbytes > SCOPE_MAX[scope]:
                    continue
                variants = [1] if op == "put_signal+wait_until" else sorted({1, spread_groups(scope, nbytes)})
                for groups in variants:
                    single = {"thread": 1 << 16, "warp": 1 << 22, "block": 64 << 20}[scope]
                    if groups == 1 and nbytes > single:
                        continue    # one thread / warp moving megabytes says nothing and takes seconds
                    iters = 20 if nbytes <= (1 << 20) else 4
                    if op == "put_nbi_x64+quiet":
                        if nbytes > (1 << 20):
                            continue
                        iters = 4
                    t = run(op, scope, nbytes, groups, iters)
                    msgs = 64 * groups if op == "put_nbi_x64+quiet" else 1
                    moved = nbytes * (64 if op == "put_nbi_x64+quiet" else 1)
                    rows.append({"op": op, "scope": scope, "bytes": nbytes, "groups": groups, "us": t / 1e3,
                                 "gbs": moved / t, "mops": msgs / t * 1e3})
        if rank == 0:
            print(f"{op}: done", flush=True)
    res = {"n_pes": world, "all_pairs": bool(args.all_pairs), "rows": rows}

    if args.host and world >= 2:
        host = {}
        buf, back = shm.zeros(1 << 17, torch.int64), shm.zeros(1 << 17, torch.int64)
        cnt = shm.zeros(1, torch.int64)
        shm.barrier_all()
        for name, fn, reps in (("putmem_1MiB", lambda: shm.putmem(buf, back, 1), 50),
                               ("getmem_1MiB", lambda: shm.getmem(back, buf, 1), 50),
                               ("putmem_8B", lambda: shm.putmem(buf[:1], back[:1], 1), 200),
                               ("atomic_fetch_add", lambda: shm.atomic_fetch_add(cnt, 1, 1), 200)):
            if rank == 0:
                for _ in range(5):
                    fn()
                t0 = time.perf_counter()
                for _ in range(reps):
                    fn()
                host[name + "_us"] = (time.perf_counter() - t0) / reps * 1e6
            shm.barrier_all()
        for _ in range(5):
            shm.barrier_all()
        t0 = time.perf_counter()
        for _ in range(100):
            shm.barrier_all()
        host["barrier_all_us"] = (time.perf_counter() - t0) / 100 * 1e6
        res["host_api"] = host

    err = shm.get_error()
    res["errors"] = err["count"]
    if rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out + ".json", "w") as f:
            json.dump(res, f, indent=1)
        with open(args.out + ".csv", "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=["op", "scope", "bytes", "groups", "us", "gbs", "mops"])
            wr.writeheader()
            wr.writerows(rows)
        print(json.dumps({"n_pes": world, "all_pairs": bool(args.all_pairs), "rows": len(rows), "errors": err["count"],
                          "host_api": res.get("host_api")}))
    shm.finalize()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
