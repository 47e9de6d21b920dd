#!/usr/bin/env python
"""Fused model blocks against their library baselines on the same GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29545 benchmarks/model_bench.py --out bench_out/model_n8.json
    python benchmarks/model_bench.py --skip tp_mlp --experts 32 --no-moe-baseline   # one rank's share of the MoE layer
                                                                                 # on one GPU (also the ncu target)

* TP MLP (default: 8192 tokens in total, d_model 8192, d_ff 28672, bf16): this package's two fused kernels
  (all-gather -> GEMM -> SwiGLU, GEMM -> reduce-scatter) against NCCL all-gather + cuBLAS + NCCL
  reduce-scatter. Roofline: the slower of FLOPs / measured GEMM peak and NVLink bytes / measured link
  bandwidth.
* MoE feed-forward (default: 256 experts, top-8, hidden 7168, intermediate 2048, 4096 tokens per rank):
  dispatch -> grouped GEMMs -> combine against an NCCL all-to-all + cuBLAS layer.

Device time with CUDA events, maximum over ranks, at least three warm-up steps; the working set of every
step (weights and activations) is far larger than L2.
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
from rocshmem_b200 import baselines  # noqa: E402
from rocshmem_b200.models import moe_ffn, tp_mlp  # noqa: E402
from rocshmem_b200.ops import gemm, moe  # noqa: E402


def timed(fn, iters, warmup=3):
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


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops_sustained"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1400.0, "fallback"


def bench_tp_mlp(args, world, rank, res):
    m_shard = args.tokens // world
    mlp = tp_mlp.TensorParallelMLP(args.d_model, args.d_ff, m_shard, seed=1)
    base = baselines.NcclTensorParallelMLP(args.d_model, args.d_ff, m_shard, seed=1)
    x = (torch.randn(m_shard, args.d_model, device="cuda") * 0.5).to(torch.bfloat16)
    mlp.input_buffer().copy_(x)
    torch.cuda.synchronize()
    shm.barrier_all()
    out = mlp.forward()
    ref = base(x)
    torch.cuda.synchronize()
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    t_fused = timed(lambda: mlp.forward(), args.iters)
    t_ag = timed(lambda: mlp.tp.ag_gemm(mlp.w_gate_up, out=mlp.h, swiglu=True), args.iters)
    t_rs = timed(lambda: mlp.tp.gemm_rs(mlp.h, mlp.w_down), args.iters)
    t_base = timed(lambda: base(x), args.iters)
    ff = args.d_ff // world
    flops = 2.0 * args.tokens * args.d_model * (2 * ff) + 2.0 * args.tokens * ff * args.d_model
    link_bytes = (world - 1) / world * args.tokens * args.d_model * 2  # per direction, each of AG and RS
    tf, src = peaks()
    roof_us = max(flops / (tf * 1e12), 2 * link_bytes / 770e9) * 1e6
    res["tp_mlp"] = {
        "tokens": args.tokens, "d_model": args.d_model, "d_ff": args.d_ff, "fused_us": t_fused, "ag_gemm_us": t_ag,
        "gemm_rs_us": t_rs, "nccl_cublas_us": t_base, "speedup": t_base / t_fused,
        "tflops_per_gpu": flops / t_fused / 1e6, "roofline_us": roof_us, "frac_of_roofline": roof_us / t_fused,
        "peak_source": src, "max_abs_diff_vs_baseline": err, "baseline_abs_max": scale,
        "gemm_errors": gemm.gemm_error_count()}
    if args.d_model % 512 == 0 and ff % 512 == 0:
        mlp8 = tp_mlp.TensorParallelMLPFp8(args.d_model, args.d_ff, m_shard, seed=1)
        out8 = mlp8(x)
        torch.cuda.synchronize()
        err8 = (out8.float() - ref.float()).abs().max().item()
        t8 = timed(lambda: mlp8(x), args.iters)
        t8_ag = timed(lambda: mlp8.tp.ag_gemm(mlp8.w1_q, mlp8.w1_s, out=mlp8.h, swiglu=True), args.iters)
        t8_rs = timed(lambda: mlp8.tp.gemm_rs(mlp8.h_q, mlp8.h_s, mlp8.w2_q, mlp8.w2_s), args.iters)
        res["tp_mlp_fp8"] = {"fused_us": t8, "ag_gemm_us": t8_ag, "gemm_rs_us": t8_rs, "speedup_vs_nccl_cublas_bf16": t_base / t8,
                             "tflops_per_gpu": flops / t8 / 1e6, "max_abs_diff_vs_bf16_baseline": err8,
                             "gemm_errors": gemm.gemm_error_count()}


def bench_moe(args, world, rank, res):
    E, K, H, I, T = args.experts, args.top_k, args.hidden, args.inter, args.moe_tokens
    cap = int(T * K * args.capacity_factor)
    layer = moe_ffn.MoEFeedForward(E, K, H, I, max_tokens=T, seed=2, pair_capacity=cap, fp8_experts=False)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    idx, w = moe.make_routing(T, E, K, seed=100 + rank, device="cuda")
    out = layer(x, idx, w)
    torch.cuda.synchronize()
    pairs = int(layer.d.recv_info[1 + 2 * world:].sum().item())
    assert pairs <= cap, (pairs, cap)
    t_layer = timed(lambda: layer(x, idx, w), args.iters)
    row = {"experts": E, "top_k": K, "hidden": H, "inter": I, "tokens_per_rank": T, "layer_us": t_layer,
           "experts_dtype": "bf16", "pairs_this_rank": pairs, "tokens_per_s_all_ranks": world * T / t_layer * 1e6}
    flops = 2.0 * pairs * H * (2 * I) + 2.0 * pairs * I * H
    row["expert_tflops_this_rank"] = flops / t_layer / 1e6
    if args.moe_baseline:
        base = baselines.NcclMoEFeedForward(E, K, H, I, seed=2)
        ref = base(x, idx, w)
        torch.cuda.synchronize()
        row["max_abs_diff_vs_baseline"] = (out.float() - ref.float()).abs().max().item()
        row["baseline_abs_max"] = ref.float().abs().max().item()
        row["nccl_cublas_us"] = timed(lambda: base(x, idx, w), max(2, args.iters // 2), warmup=2)
        row["speedup"] = row["nccl_cublas_us"] / t_layer
    stages = {}
    layer(x, idx, w, stage_us=stages)
    row["stage_us_rank0"] = stages
    layer.destroy()
    if H % 512 == 0 and I % 512 == 0:
        layer8 = moe_ffn.MoEFeedForward(E, K, H, I, max_tokens=T, seed=2, pair_capacity=cap, fp8_experts=True)
        out8 = layer8(x, idx, w)
        torch.cuda.synchronize()
        stages8 = {}
        layer8(x, idx, w, stage_us=stages8)
        row["fp8_experts_stage_us_rank0"] = stages8
        row["fp8_experts_max_abs_diff_vs_bf16_experts"] = (out8.float() - out.float()).abs().max().item()
        row["fp8_experts_layer_us"] = timed(lambda: layer8(x, idx, w), args.iters)
        row["fp8_experts_tokens_per_s_all_ranks"] = world * T / row["fp8_experts_layer_us"] * 1e6
        row["fp8_experts_tflops_this_rank"] = flops / row["fp8_experts_layer_us"] / 1e6
        if args.moe_baseline:
            row["fp8_experts_speedup"] = row["nccl_cublas_us"] / row["fp8_experts_layer_us"]
        layer8.destroy()
    row["gemm_errors"] = gemm.gemm_error_count()
    res["moe_ffn"] = row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bench_out/model_bench.json")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=8192)
    ap.add_argument("--d-ff", type=int, default=28672)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--moe-tokens", type=int, default=4096)
    ap.add_argument("--capacity-factor", type=float, default=1.5)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip", default="", help="comma list of: tp_mlp, moe")
    ap.add_argument("--no-moe-baseline", dest="moe_baseline", action="store_false")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29547")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    shm.init(heap_size=24 << 30, device=local)
    res = {"n_gpus": world}
    skip = set(args.skip.split(","))
    if "tp_mlp" not in skip:
        bench_tp_mlp(args, world, rank, res)
    if "moe" not in skip:
        bench_moe(args, world, rank, res)
    err = shm.get_error()
    res["runtime_errors"] = err["count"]
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)
        print(json.dumps(res))
    torch.cuda.synchronize()
    shm.barrier_all()
    shm.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
