#!/usr/bin/env python
"""tcgen05 GEMM kernels of this package against cuBLAS (``torch.matmul``) on one GPU.

    python benchmarks/gemm_bench.py --out bench_out/gemm_bench.json          # the table
    python benchmarks/gemm_bench.py --profile                                   # one small shape, few launches
    python benchmarks/gemm_bench.py --profile-fp8                               # the same for the e4m3 kernel
    ncu --set full --clock-control none -k regex:gemm_bf16_kernel -c 2 -o bench_out/gemm \
        python benchmarks/gemm_bench.py --profile

Shapes are the per-rank GEMMs of the tensor-parallel MLP (8192 tokens, d_model 8192, d_ff 28672 over 8 or
2 ranks) and of the MoE experts (hidden 7168, intermediate 2048, 32 experts per rank, 32768 rows).
Device time with CUDA events after three warm-up launches; a 256 MB buffer is written between timed
launches so that no operand is left in L2 by the previous one. Fractions are of the measured cuBLAS bf16
peak (burst figure, the kernels are timed in isolation).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rocshmem_b200.ops import gemm  # noqa: E402


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(iters):
        flush.add_(1)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    return total / iters * 1e3


def peak():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--profile-fp8", action="store_true")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dev = "cuda"
    if args.profile:
        m, n, k = 4096, 4096, 8192  # 64 + 64 + 32 MB of operands, a third of a millisecond
        a = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
        b = (torch.randn(n, k, device=dev) * 0.5).to(torch.bfloat16)
        for _ in range(3):
            c = gemm.gemm_bf16(a, b)
        torch.cuda.synchronize()
        assert gemm.gemm_error_count() == 0
        print("profile run done", float(c[0, 0]))
        return
    if args.profile_fp8:
        from rocshmem_b200.ops import moe
        m, n, k = 4096, 4096, 8192
        a = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
        b = (torch.randn(n, k, device=dev) * 0.5).to(torch.bfloat16)
        a_q, a_s = moe.fp8_quantize_1x128(a)
        b_q, b_s = gemm.quantize_weight_128x128(b)
        for _ in range(3):
            c = gemm.gemm_fp8_blockscaled(a_q, a_s, b_q, b_s)
        torch.cuda.synchronize()
        assert gemm.gemm_error_count() == 0
        print("fp8 profile run done", float(c[0, 0]))
        return
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    pk, src = peak()
    rows = []
    shapes = [(8192, 3584, 8192), (8192, 7168, 8192), (8192, 8192, 3584), (8192, 28672, 8192), (8192, 8192, 14336),
              (4096, 4096, 4096), (1024, 8192, 8192)]
    for m, n, k in shapes:
        a = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
        b = (torch.randn(n, k, device=dev) * 0.5).to(torch.bfloat16)
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        t_own = timed(lambda: gemm.gemm_bf16(a, b, out=c), args.iters, flush)
        ref = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        bt = b.t()
        t_lib = timed(lambda: torch.matmul(a, bt, out=ref), args.iters, flush)
        diff = (c.float() - ref.float()).abs().max().item()
        fl = 2.0 * m * n * k
        rows.append({"op": "gemm_bf16", "m": m, "n": n, "k": k, "us": t_own, "tflops": fl / t_own / 1e6,
                     "frac_of_peak": fl / t_own / 1e6 / pk, "cublas_us": t_lib, "cublas_tflops": fl / t_lib / 1e6,
                     "max_abs_diff_vs_cublas": diff})
        del a, b, c, ref
    # grouped: 32 experts, 1024 rows each
    G, rows_g, H, I = 32, 1024, 7168, 2048
    off = torch.arange(G + 1, dtype=torch.int32, device=dev) * rows_g
    xs = (torch.randn(G * rows_g, H, device=dev) * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(G, 2 * I, H, device=dev) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(G, H, I, device=dev) * I ** -0.5).to(torch.bfloat16)
    h = torch.empty(G * rows_g, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(G * rows_g, H, dtype=torch.bfloat16, device=dev)
    t1 = timed(lambda: gemm.grouped_gemm_bf16(xs, w13, off, swiglu=True, out=h), args.iters, flush)
    t2 = timed(lambda: gemm.grouped_gemm_bf16(h, w2, off, out=y), args.iters, flush)
    f1, f2 = 2.0 * G * rows_g * H * 2 * I, 2.0 * G * rows_g * I * H
    rows.append({"op": "grouped_gemm_swiglu", "groups": G, "rows": G * rows_g, "n": 2 * I, "k": H, "us": t1,
                 "tflops": f1 / t1 / 1e6, "frac_of_peak": f1 / t1 / 1e6 / pk})
    rows.append({"op": "grouped_gemm", "groups": G, "rows": G * rows_g, "n": H, "k": I, "us": t2,
                 "tflops": f2 / t2 / 1e6, "frac_of_peak": f2 / t2 / 1e6 / pk})
    del xs, w13, w2, h, y
    # block-scaled e4m3 (1 x 128 activation scales, 128 x 128 weight scales); the fraction is still of the
    # bf16 peak, so values above 1 are expected
    from rocshmem_b200.ops import moe
    for m, n, k in [(8192, 7168, 8192), (8192, 8192, 3584), (8192, 28672, 8192)]:
        a = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
        b = (torch.randn(n, k, device=dev) * 0.5).to(torch.bfloat16)
        a_q, a_s = moe.fp8_quantize_1x128(a)
        b_q, b_s = gemm.quantize_weight_128x128(b)
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        t8 = timed(lambda: gemm.gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, out=c), args.iters, flush)
        fl = 2.0 * m * n * k
        rows.append({"op": "gemm_fp8_blockscaled", "m": m, "n": n, "k": k, "us": t8, "tflops": fl / t8 / 1e6,
                     "frac_of_bf16_peak": fl / t8 / 1e6 / pk})
        del a, b, a_q, a_s, b_q, b_s, c
    res = {"peak_tflops": pk, "peak_source": src, "gemm_errors": gemm.gemm_error_count(), "rows": rows}
    for r in rows:
        print(json.dumps(r))
    if args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)


if __name__ == "__main__":
    main()
