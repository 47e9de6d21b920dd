#!/usr/bin/env python
"""Runs the functional driver over a matrix of tests, launch shapes and message sizes and collects the rows in one
CSV file (the role of the reference's scripts/functional_tests/driver.sh, which walks a table of test name, ranks,
work-groups, threads and maximum message size).

    python benchmarks/run_matrix.py --gpus 2                 # one process per GPU
    python benchmarks/run_matrix.py --local-pes 2            # two PEs on one GPU
    python benchmarks/run_matrix.py --dry-run                # print the commands only
    python benchmarks/run_matrix.py --only put,allreduce --out bench_out/matrix.csv

Every case is one run of ``benchmarks/functional_driver.py`` started through ``rocshmem_b200.launch``; a case that
fails or times out is recorded as such and the walk continues. Launch shapes follow the hardware: blocks from one to
one per SM pair, threads from one warp to a full block.
"""
from __future__ import annotations

import argparse
import csv
import io
import os
import sys
from typing import List, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

# (test, blocks, threads, max bytes). Device-timed point-to-point tests walk launch shapes; library collectives
# choose their own grids, so they only walk sizes.
MATRIX: List[Tuple[str, int, int, int]] = (
    [("put", b, t, s) for (b, t, s) in ((1, 32, 1 << 20), (1, 1024, 1 << 20), (8, 256, 1 << 22), (32, 512, 1 << 24),
                                        (74, 512, 1 << 26), (128, 1024, 1 << 26))]
    + [("get", b, t, s) for (b, t, s) in ((1, 32, 1 << 20), (1, 1024, 1 << 20), (8, 256, 1 << 22), (32, 512, 1 << 24),
                                          (74, 512, 1 << 26), (128, 1024, 1 << 26))]
    + [(name, b, t, 8) for name in ("amo_fadd", "amo_finc", "amo_add", "amo_fcswap")
       for (b, t) in ((1, 1), (1, 64), (8, 128), (64, 256))]
    # one call per thread / warp / block of one block (the reference's launch shapes of its single-work-group runs)
    + [(f"{op}_{scope}", 1, t, 1 << 20) for op in ("put", "put_nbi", "get", "get_nbi") for scope in ("thread", "wave", "wg")
       for t in (64, 1024)]
    + [(name, 1, 256, 1 << 16) for name in ("p", "g", "ctx_put_thread", "ctx_get_thread")]
    + [(name, 8, 128, 8) for name in ("amo_fetch", "amo_inc", "amo_set", "amo_swap", "amo_fetch_and", "amo_fetch_or",
                                      "amo_fetch_xor", "amo_and", "amo_or", "amo_xor")]
    + [(name, 1, 256, 1 << 20) for name in ("put_signal", "put_signal_wave", "put_signal_wg")]
    + [("pingpong", 1, 32, 4), ("pingall", 1, 32, 8), ("barrier", 1, 64, 0), ("barrier", 1, 1024, 0)]
    + [(name, 1, 512, 1 << 26) for name in ("allreduce", "broadcast", "fcollect", "alltoall")]
)


def command(case: Tuple[str, int, int, int], local_pes: int) -> List[str]:
    test, blocks, threads, max_bytes = case
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "functional_driver.py"), "-a", test, "-w", str(blocks), "-z",
           str(threads), "-s", str(max(8, max_bytes))]
    if local_pes:
        cmd += ["--local-pes", str(local_pes)]
    return cmd


def parse_rows(text: str):
    """The driver's table: size, messages, latency (us), bandwidth (GB/s), message rate."""
    for line in text.splitlines():
        line = line.split("] ", 1)[-1] if line.startswith("[") else line     # the launcher's rank prefix
        parts = line.split()
        if len(parts) == 5 and parts[0].isdigit():
            try:
                yield int(parts[0]), int(parts[1]), float(parts[2]), float(parts[3]), float(parts[4])
            except ValueError:
                continue


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1, help="processes to start, one per GPU")
    ap.add_argument("--local-pes", type=int, default=0, help="PEs per process on one GPU (with --gpus 1)")
    ap.add_argument("--only", default="", help="comma-separated test names")
    ap.add_argument("--out", default=os.path.join("bench_out", "matrix.csv"))
    ap.add_argument("--timeout", type=float, default=300.0, help="seconds per case")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    if args.gpus == 1 and not args.local_pes:
        args.local_pes = 2                       # the tests need a peer
    only = {t for t in args.only.split(",") if t}
    cases = [c for c in MATRIX if not only or c[0] in only]
    if args.dry_run:
        for c in cases:
            print(f"python -m rocshmem_b200.launch -n {args.gpus} -- " + " ".join(command(c, args.local_pes)))
        return 0
    from rocshmem_b200 import launch
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    failed = 0
    with open(args.out, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["test", "blocks", "threads", "size_bytes", "messages", "latency_us", "bandwidth_gbs", "msg_per_s", "status"])
        for c in cases:
            buf = io.StringIO()
            rc = launch.launch(command(c, args.local_pes), args.gpus, timeout_s=args.timeout, out=buf)
            rows = list(parse_rows(buf.getvalue()))
            status = "ok" if rc == 0 and rows else ("timeout" if rc == 124 else f"failed ({rc})")
            if status != "ok":
                failed += 1
                w.writerow([c[0], c[1], c[2], "", "", "", "", "", status])
            for size, msgs, lat, bw, rate in rows:
                w.writerow([c[0], c[1], c[2], size, msgs, lat, bw, rate, status])
            f.flush()
            print(f"{c[0]:10s} blocks {c[1]:4d} threads {c[2]:5d}: {status}, {len(rows)} rows", flush=True)
    print(f"wrote {args.out}; {failed} of {len(cases)} cases failed")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
