#!/usr/bin/env python
"""Command-line performance driver in the style of the reference's ``rocshmem_example_driver``.

    python benchmarks/functional_driver.py -a put -s 1048576 --local-pes 2          # two PEs on one GPU
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/functional_driver.py -a allreduce -s 67108864                    # one PE per GPU

``-a`` selects the test by name, or by the reference's number (tests/functional_tests/tester.hpp:36-96) where
the test has a timed form here:

* put, get: block-scope RMA from PE 0 to PE 1, timed on the device;
* put_thread / put_nbi_thread / get_thread / get_nbi_thread / p / g, the same with ``_wave`` and ``_wg``, and
  ``ctx_`` + any of them for a context created inside the kernel: every PE moves the message to its right-hand
  neighbour with one call per thread, warp or block (a kernel per call, timed with CUDA events, so the figure
  includes the launch and the closing barrier);
* amo_fadd, amo_finc, amo_fetch, amo_fcswap, amo_cswap, amo_add, amo_inc, amo_set, amo_swap, amo_fetch_and /
  _or / _xor, amo_and / _or / _xor: int64 atomics on PE 0 from every thread of every PE;
* put_signal, put_signal_wave, put_signal_wg (and their ``_nbi`` numbers), signal_fetch: a message with a signal
  to the right-hand neighbour, a wait for the own signal and a ``signal_fetch``;
* pingpong (signal round trips), pingall (the wait_until_all / any / some family), barrier, sync (device barriers),
  shmem_ptr (a store through ``rocshmem_ptr`` of the neighbour), ctx_infra (creating and destroying ten contexts);
* the library collectives allreduce, broadcast, fcollect, alltoall (timed with CUDA events, maximum over PEs).

Message sizes double from ``-m`` to ``-s``; every row prints the columns of the reference's harness
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

AMO = {"amo_fadd": 0, "amo_finc": 1, "amo_add": 2, "amo_inc": 3, "amo_fcswap": 4, "amo_cswap": 4, "amo_fetch": 5,
       "amo_set": 6, "amo_swap": 7, "amo_fetch_and": 8, "amo_and": 9, "amo_fetch_or": 10, "amo_or": 11,
       "amo_fetch_xor": 12, "amo_xor": 13}

# rma_kernel of the test module: operation and scope codes
RMA_OPS = {"put": 0, "put_nbi": 1, "get": 2, "get_nbi": 3, "p": 4, "g": 5}
RMA_SCOPES = {"thread": 0, "wave": 1, "wg": 2}


def rma_form(name: str):
    """(operation, scope, use_ctx) for names like put_nbi_wave, ctx_get_thread, p; None for other tests."""
    use_ctx = name.startswith("ctx_")
    base = name[4:] if use_ctx else name
    if base in ("p", "g"):
        return RMA_OPS[base], 0, int(use_ctx)
    op, _, scope = base.rpartition("_")
    if op in RMA_OPS and op not in ("p", "g") and scope in RMA_SCOPES:
        return RMA_OPS[op], RMA_SCOPES[scope], int(use_ctx)
    return None


SIGNAL_SCOPES = {"put_signal": 0, "put_signal_wave": 1, "put_signal_wg": 2, "signal_fetch": 0}

# The reference selects tests by number (enum TestType, tests/functional_tests/tester.hpp:36-96). Numbers whose test
# has a timed form here map to its name; the functional content of all of them is covered by the pytest suite
# (tests/test_gpu_device_api.py), which is where the others point.
REFERENCE_NUMBERS = {
    0: "get_thread", 1: "get_nbi_thread", 2: "put_thread", 3: "put_nbi_thread", 5: "amo_fadd", 6: "amo_finc",
    7: "amo_fetch", 8: "amo_fcswap", 9: "amo_add", 10: "amo_inc", 11: "amo_cswap", 13: "pingpong", 15: "barrier",
    16: "barrier", 17: "barrier", 19: "fcollect", 20: "alltoall", 22: "shmem_ptr", 23: "p", 24: "g", 25: "get_wg", 26: "get_nbi_wg",
    27: "put_wg", 28: "put_nbi_wg", 29: "get_wave", 30: "get_nbi_wave", 31: "put_wave", 32: "put_nbi_wave",
    33: "broadcast", 34: "allreduce", 35: "ctx_get_thread", 36: "ctx_get_nbi_thread", 37: "ctx_put_thread",
    38: "ctx_put_nbi_thread", 39: "ctx_infra", 41: "amo_set", 42: "amo_swap", 43: "amo_fetch_and", 44: "amo_fetch_or",
    45: "amo_fetch_xor", 46: "amo_and", 47: "amo_or", 48: "amo_xor", 49: "pingall", 50: "put_signal",
    51: "put_signal_wg", 52: "put_signal_wave", 53: "put_signal", 54: "put_signal_wg", 55: "put_signal_wave",
    56: "signal_fetch", 57: "signal_fetch", 58: "signal_fetch",
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
    elif rma_form(args.test) is not None:
        if n < 2:
            raise SystemExit("RMA tests need at least two PEs")
        op, scope, use_ctx = rma_form(args.test)
        src, dst = shm.zeros(args.max_bytes, torch.uint8), shm.zeros(args.max_bytes, torch.uint8)
        for size in sizes:
            size = max(size, 8 * args.threads) if op >= 4 else size       # p / g move 8-byte elements
            us = event_time(lambda: k.rma(op, scope, dst.data_ptr(), src.data_ptr(), size, 1, use_ctx, args.threads, stream),
                            args.loop, args.skip)
            if not quiet:
                row(size, args.loop, us)
    elif args.test in SIGNAL_SCOPES:
        if n < 2:
            raise SystemExit("signal tests need at least two PEs")
        src, dst = shm.zeros(args.max_bytes, torch.uint8), shm.zeros(args.max_bytes, torch.uint8)
        sig, fetched = shm.zeros(1, torch.int64), shm.zeros(2, torch.int64)
        scope = SIGNAL_SCOPES[args.test]
        for size in sizes:
            size = max(size, args.threads)        # a thread's share is size / threads bytes
            # SET of 1 with a wait for 1: every launch after the first finds the signal already there, so the
            # figure is the cost of the message, the signal, the check and the closing barrier
            us = event_time(lambda: k.signal(scope, 0, dst.data_ptr(), src.data_ptr(), size, sig.data_ptr(), 1, 1,
                                             fetched.data_ptr(), args.threads, stream), args.loop, args.skip)
            if not quiet:
                row(size, args.loop, us)
    elif args.test == "shmem_ptr":
        buf = shm.zeros(16, torch.uint8)
        us = event_time(lambda: k.shmem_ptr(buf.data_ptr(), 4, stream), args.loop, args.skip)
        if not quiet:
            row(1, args.loop, us)
    elif args.test == "ctx_infra":
        out = shm.zeros(1, torch.int32)
        us = event_time(lambda: k.ctx_exhaust(10, out.data_ptr(), stream), args.loop, args.skip)
        if not quiet:
            row(0, args.loop * 10, us)
    elif args.test == "pingall":
        slots, result = shm.zeros(max(n, 8), torch.int64), shm.zeros(8, torch.int64)
        us = event_time(lambda: k.pingall(slots.data_ptr(), result.data_ptr(), stream), args.loop, args.skip)
        if not quiet:
            row(8, args.loop * n, us)
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
