#!/usr/bin/env python
"""Command-line performance driver in the style of the reference's ``rocshmem_example_driver``.

    python benchmarks/functional_driver.py -a put -s 1048576 --local-pes 2          # two PEs on one GPU
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/functional_driver.py -a allreduce -s 67108864                    # one PE per GPU

``-a`` selects the test by name, or by the reference's number (tests/functional_tests/tester.hpp:36-96) where
the test has a timed form here:
put, get (block-scope RMA from PE 0 to PE 1, timed on the device), amo_fadd / amo_finc / amo_fcswap / amo_add
(int64 atomics on PE 0 from every PE), pingpong (signal round trips), barrier (device barrier_all), and the
library collectives allreduce, broadcast, fcollect, alltoall (timed with CUDA events on the host, maximum over
PEs). Message sizes double from ``-m`` to ``-s``; every row prints the columns of the reference's harness
(tests/functional_tests/tester.cpp:488-531): size in bytes, timed messages, latency in microseconds,
bandwidth in GB/s (10^9 bytes) and message rate.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200 import _native  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402

AMO = {"amo_fadd": 0, "amo_finc": 1, "amo_add": 2, "amo_fcswap": 4}

# The reference selects tests by number (enum TestType, tests/functional_tests/tester.hpp:36-96). Numbers whose test
# has a timed form here map to its name; the functional content of all of them is covered by the pytest suite
# (tests/test_gpu_device_api.py), which is where the others point.
REFERENCE_NUMBERS = {
    0: "get", 1: "get", 2: "put", 3: "put", 5: "amo_fadd", 6: "amo_finc", 8: "amo_fcswap", 9: "amo_add",
    13: "pingpong", 15: "barrier", 16: "barrier", 19: "fcollect", 20: "alltoall", 25: "get", 26: "get", 27: "put",
    28: "put", 33: "broadcast", 34: "allreduce",
}
REFERENCE_NAMES = [
    "Get", "GetNBI", "Put", "PutNBI", "GetSwarm", "AMO_FAdd", "AMO_FInc", "AMO_Fetch", "AMO_FCswap", "AMO_Add", "AMO_Inc",
    "AMO_Cswap", "Init", "PingPong", "RandomAccess", "BarrierAll", "SyncAll", "Sync", "Collect", "TeamFCollect",
    "TeamAllToAll", "AllToAlls", "ShmemPtr", "P", "G", "WGGet", "WGGetNBI", "WGPut", "WGPutNBI", "WAVEGet", "WAVEGetNBI",
    "WAVEPut", "WAVEPutNBI", "TeamBroadcast", "TeamReduction", "TeamCtxGet", "TeamCtxGetNBI", "TeamCtxPut",
    "TeamCtxPutNBI", "TeamCtxInfra", "PutNBIMR", "AMO_Set", "AMO_Swap", "AMO_FetchAnd", "AMO_FetchOr", "AMO_FetchXor",
    "AMO_And", "AMO_Or", "AMO_Xor", "PingAll", "PutSignal", "WGPutSignal", "WAVEPutSignal", "PutSignalNBI",
    "WGPutSignalNBI", "WAVEPutSignalNBI", "SignalFetch", "WGSignalFetch", "WAVESignalFetch",
]


def resolve_test(selector: str) -> str:
    """A test name as it is, or the name for one of the reference's test numbers (0 .. 58)."""
    if not selector.lstrip("-").isdigit():
        return selector
    number = int(selector)
    if not 0 <= number < len(REFERENCE_NAMES):
        raise SystemExit(f"test numbers run from 0 to {len(REFERENCE_NAMES) - 1}")
    if number not in REFERENCE_NUMBERS:
        raise SystemExit(f"test {number} ({REFERENCE_NAMES[number]}TestType) has no timed form in this driver; its "
                         "checks are part of the pytest suite: python -m pytest tests/test_gpu_device_api.py -m gpu")
    return REFERENCE_NUMBERS[number]


def header():
    print(f"{'Size (B)':>12} {'# msgs':>10} {'Latency (us)':>14} {'Bandwidth (GB/s)':>18} {'Msg rate (msg/s)':>18}")


def row(size, msgs, us_total):
    lat = us_total / max(1, msgs)
    print(f"{size:>12} {msgs:>10} {lat:>14.3f} {size * msgs / us_total / 1e3:>18.3f} {msgs / us_total * 1e6:>18.0f}", flush=True)


def event_time(fn, iters, skip):
    for _ in range(skip):
        fn()
    torch.cuda.synchronize()
    shm.barrier_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-a", "--test", default="put")
    ap.add_argument("-w", "--blocks", type=int, default=1, help="thread blocks (work-groups)")
    ap.add_argument("-z", "--threads", type=int, default=512, help="threads per block")
    ap.add_argument("-m", "--min-bytes", type=int, default=8)
    ap.add_argument("-s", "--max-bytes", type=int, default=1 << 20)
    ap.add_argument("--loop", type=int, default=10)
    ap.add_argument("--skip", type=int, default=10)
    ap.add_argument("--local-pes", type=int, default=0, help="PEs hosted by this process on one GPU (0: one per process)")
    args = ap.parse_args()
    args.test = resolve_test(args.test)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    kw = {"n_local": args.local_pes} if args.local_pes else {}
    shm.init(heap_size=max(1 << 30, 4 * args.max_bytes * max(2, args.local_pes)), device=local, **kw)
    k = _native.load_test_kernels()
    n, me = shm.n_pes(), shm.my_pe()
    stream = torch.cuda.current_stream().cuda_stream
    quiet = me != 0
    if not quiet:
        print(f"# test {args.test}, {n} PEs, {args.blocks} block(s) x {args.threads} threads, loop {args.loop}, skip {args.skip}")
        header()
    sizes = []
    s = args.min_bytes
    while s <= args.max_bytes:
        sizes.append(s)
        s *= 2
    if args.test in ("put", "get"):
        if n < 2:
            raise SystemExit("put / get need at least two PEs")
        src, dst = shm.zeros(args.max_bytes, torch.uint8), shm.zeros(args.max_bytes, torch.uint8)
        ns = shm.zeros(256, torch.int64)
        for size in sizes:
            blocks = max(1, min(args.blocks, size // 16))
            for iters in (args.skip, args.loop):
                k.bw(0 if args.test == "put" else 1, dst.data_ptr(), src.data_ptr(), size, 1, iters, ns.data_ptr(), blocks,
                     args.threads, stream)
                torch.cuda.synchronize()
                shm.barrier_all()
            if not quiet:
                row(size, args.loop, float(ns[:blocks].max().item()) / 1e3)
    elif args.test in AMO:
        target, ret = shm.zeros(1, torch.int64), shm.zeros(args.blocks * args.threads, torch.int64)
        us = event_time(lambda: k.amo(AMO[args.test], target.data_ptr(), ret.data_ptr(), args.loop, args.blocks, args.threads,
                                      stream), 1, 1)
        if not quiet:
            row(8, args.loop * args.blocks * args.threads, us)
    elif args.test == "pingpong":
        flag, ns = shm.zeros(1, torch.int32), shm.zeros(1, torch.int64)
        iters = args.loop * 100
        k.pingpong(flag.data_ptr(), iters, ns.data_ptr(), stream)
        torch.cuda.synchronize()
        shm.barrier_all()
        if not quiet:
            row(4, iters, float(ns[0].item()) / 1e3)
    elif args.test == "barrier":
        slots, errors = shm.zeros(64, torch.int64), shm.zeros(1, torch.int32)
        rounds = args.loop * 10
        us = event_time(lambda: k.barrier_stress(slots.data_ptr(), rounds, errors.data_ptr(), args.threads, stream), 1, 1)
        if not quiet:
            row(0, rounds, us)
    elif args.test in ("allreduce", "broadcast", "fcollect", "alltoall"):
        elems = args.max_bytes // 4
        src, dst = shm.zeros(elems * (n if args.test == "alltoall" else 1), torch.float32), shm.zeros(elems * n, torch.float32)
        src.normal_()
        for size in sizes:
            e = max(1, size // 4)
            fn = {"allreduce": lambda: coll.allreduce_async(dst[:e], src[:e], shm.OP_SUM),
                  "broadcast": lambda: coll.broadcast_async(dst[:e], src[:e], 0),
                  "fcollect": lambda: coll.fcollect_async(dst[:e * n], src[:e]),
                  "alltoall": lambda: coll.alltoall_async(dst[:e * n], src[:e * n])}[args.test]
            us = event_time(fn, args.loop, args.skip)
            if not quiet:
                row(e * 4, args.loop, us)
    else:
        raise SystemExit(f"unknown test {args.test!r}")
    err = shm.get_error()
    torch.cuda.synchronize()
    shm.barrier_all()
    shm.finalize()
    if err["count"]:
        print("runtime error record:", err)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
