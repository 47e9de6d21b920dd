#!/usr/bin/env python
"""Every library kernel family once (or a few times) on ONE GPU, at sizes that exceed the 126 MB L2 but stay small:
a quick timing table, and the target of profiler captures (one kernel family per capture, selected by name).

    python benchmarks/kernel_tour.py                          # all families, CUDA-event times
    python benchmarks/kernel_tour.py --only collectives       # comma list of: collectives, ep, moe, tp
    ncu --set full --clock-control none -k regex:allreduce_two_shot -c 2 -o <out> \
        python benchmarks/kernel_tour.py --only collectives --reps 1

Families:
  collectives  two PEs on the one GPU (one cooperative launch per call, so the peer paths run over the local
               mapping): allreduce (flag-in-word, one-shot, two-shot), fcollect / alltoall / broadcast push kernels
  ep           dispatch and combine, fixed shares and pair hand-out, and the low-latency pair (one PE)
  moe          the grouped GEMMs of the MoE layer: gathered bf16 rows with SwiGLU, scatter-add, and their
               block-scaled forms (gathered e4m3 rows, quantising epilogue) (32 experts x ~1024 rows, hidden 7168, intermediate 2048)
  tp           all-gather -> GEMM and GEMM -> reduce-scatter on a team of one (the tensor-core side of the fused
               kernels; the NVLink side needs several GPUs and is timed by benchmarks/model_bench.py)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402
from rocshmem_b200.ops import gemm, moe  # noqa: E402


def timed(fn, reps, flush):
    fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / reps * 1e3


def tour_collectives(reps, flush, rows):
    shm.init(n_local=2, heap_size="2G", device=0)
    try:
        n = 64 << 20   # bytes per PE: source + dest of both PEs = 256 MB
        src, dst = shm.zeros(n // 2, torch.bfloat16), shm.zeros(n, torch.bfloat16)
        for l in range(2):
            shm.local_view(src, l).normal_()
        torch.cuda.synchronize()
        small = 512
        for name, fn in (
            ("allreduce_ll 1 KiB", lambda: coll.allreduce_async(dst[:small], src[:small], algo=shm.ALLREDUCE_LL)),
            ("allreduce_one_shot 256 KiB", lambda: coll.allreduce_async(dst[:1 << 17], src[:1 << 17], algo=shm.ALLREDUCE_ONE_SHOT)),
            ("allreduce_two_shot 64 MiB", lambda: coll.allreduce_async(dst[:n // 2], src, algo=shm.ALLREDUCE_TWO_SHOT)),
            ("fcollect 64 MiB per PE", lambda: coll.fcollect_async(dst, src)),
            ("alltoall 32 MiB per peer", lambda: coll.alltoall_async(dst[:n // 2], src)),
            ("broadcast 64 MiB", lambda: coll.broadcast_async(dst[:n // 2], src, 0)),
        ):
            rows.append({"family": "collectives", "kernel": name, "us": timed(fn, reps, flush)})
        assert shm.get_error()["count"] == 0
    finally:
        torch.cuda.synchronize()
        shm.finalize()


def tour_ep(reps, flush, rows):
    shm.init(n_local=1, heap_size="3G", device=0)
    try:
        T, H, E, K = 8192, 7168, 256, 8
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        idx, w = moe.make_routing(T, E, K, 3, "cuda")
        out = torch.empty_like(x)
        for label, kw in (("fixed shares", dict(dynamic=False)), ("pair hand-out", dict(dynamic=True)),
                          ("pair hand-out + expert layout", dict(dynamic=True, expert_layout=True))):
            d = moe.EpDispatcher(E, K, H, T, **kw)
            y = d.result_buffer()
            rows.append({"family": "ep", "kernel": f"dispatch, {label}, {T} tokens", "us": timed(lambda: d.dispatch(x, idx, w), reps, flush)})
            rows.append({"family": "ep", "kernel": f"combine, {label}, {T} tokens", "us": timed(lambda: d.combine(y, idx, w, T, out=out), reps, flush)})
            d.destroy()
        d = moe.EpDispatcher(E, K, H, 128, low_latency=True)
        y = d.result_buffer()
        rows.append({"family": "ep", "kernel": "low-latency dispatch, 128 tokens", "us": timed(lambda: d.dispatch(x[:128], idx[:128], w[:128]), reps, flush)})
        rows.append({"family": "ep", "kernel": "low-latency combine, 128 tokens", "us": timed(lambda: d.combine(y, idx[:128], w[:128], 128, out=out[:128]), reps, flush)})
        d.destroy()
        assert shm.get_error()["count"] == 0
    finally:
        torch.cuda.synchronize()
        shm.finalize()


def tour_moe(reps, flush, rows):
    G, H, I, src_rows = 32, 7168, 2048, 22000
    g = torch.Generator(device="cuda").manual_seed(7)
    sizes = torch.randint(900, 1150, (G,), generator=g, device="cuda")
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), sizes.cumsum(0)]).to(torch.int32)
    pairs = int(offsets[-1])
    row_index = torch.randint(0, src_rows, (pairs,), generator=g, device="cuda", dtype=torch.int32)
    weights = torch.rand(pairs, generator=g, device="cuda")
    xq, xs = moe.fp8_quantize_1x128((torch.randn(src_rows, H, generator=g, device="cuda") * 0.5).to(torch.bfloat16))
    w13 = (torch.randn(G, 2 * I, H, generator=g, device="cuda") * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(G, H, I, generator=g, device="cuda") * I ** -0.5).to(torch.bfloat16)
    h = torch.empty(pairs, I, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(src_rows, H, dtype=torch.bfloat16, device="cuda")
    f1, f2 = 2.0 * pairs * H * 2 * I, 2.0 * pairs * I * H

    def add(name, us, flops):
        rows.append({"family": "moe", "kernel": name, "us": us, "tflops": flops / us / 1e6})

    xb = moe.fp8_dequantize_1x128(xq, xs)
    add("grouped gate/up, gathered bf16 rows, SwiGLU", timed(lambda: gemm.grouped_gemm_bf16_gathered(xb, row_index, w13, offsets, swiglu=True, out=h), reps, flush), f1)
    del xb
    add("grouped down, scatter-add epilogue", timed(lambda: gemm.grouped_gemm_bf16_scatter_add(h, w2, offsets, row_index, y, weights=weights), reps, flush), f2)
    w13q, w13s = gemm.quantize_weight_128x128(w13)
    w2q, w2s = gemm.quantize_weight_128x128(w2)
    del w13, w2
    hq = torch.empty(pairs, I, dtype=torch.uint8, device="cuda")
    hs = torch.empty(pairs, I // 128, dtype=torch.float32, device="cuda")
    add("block-scaled grouped gate/up, gathered e4m3, SwiGLU + quantise", timed(lambda: gemm.grouped_gemm_fp8_swiglu_quant(xq.view(torch.uint8), xs, w13q, w13s, offsets, hq, hs, row_index=row_index), reps, flush), f1)
    add("block-scaled grouped down, scatter-add epilogue", timed(lambda: gemm.grouped_gemm_fp8_scatter_add(hq, hs, w2q, w2s, offsets, row_index, y, weights=weights), reps, flush), f2)
    assert gemm.gemm_error_count() == 0


def tour_tp(reps, flush, rows):
    shm.init(n_local=1, heap_size="4G", device=0)
    try:
        m, d_model, ff = 4096, 8192, 3584
        tp = gemm.TensorParallelLinear(m)
        x = (torch.randn(m, d_model, device="cuda") * 0.5).to(torch.bfloat16)
        w1 = (torch.randn(2 * ff, d_model, device="cuda") * 0.02).to(torch.bfloat16)
        w2 = (torch.randn(d_model, ff, device="cuda") * 0.02).to(torch.bfloat16)
        tp.ag_input(d_model).copy_(x)
        h = torch.empty(m, ff, dtype=torch.bfloat16, device="cuda")
        us = timed(lambda: tp.ag_gemm(w1, out=h, swiglu=True), reps, flush)
        rows.append({"family": "tp", "kernel": f"all-gather -> GEMM + SwiGLU, {m} x {2 * ff} x {d_model}", "us": us,
                     "tflops": 2.0 * m * 2 * ff * d_model / us / 1e6})
        us = timed(lambda: tp.gemm_rs(h, w2), reps, flush)
        rows.append({"family": "tp", "kernel": f"GEMM -> reduce-scatter, {m} x {d_model} x {ff}", "us": us,
                     "tflops": 2.0 * m * d_model * ff / us / 1e6})
        assert gemm.gemm_error_count() == 0 and shm.get_error()["count"] == 0
    finally:
        torch.cuda.synchronize()
        shm.finalize()


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--only", default="collectives,ep,moe,tp")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    only = set(args.only.split(","))
    if "collectives" in only:
        tour_collectives(args.reps, flush, rows)
    if "ep" in only:
        tour_ep(args.reps, flush, rows)
    if "moe" in only:
        tour_moe(args.reps, flush, rows)
    if "tp" in only:
        tour_tp(args.reps, flush, rows)
    for r in rows:
        print(json.dumps({k: (round(v, 1) if isinstance(v, float) else v) for k, v in r.items()}))
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
