#!/usr/bin/env python
"""Headline benchmark: DeepEP-style expert-parallel dispatch + combine on N GPUs of one node.

One step = for every rank, dispatch 4096 bf16 tokens (hidden 7168) to the ranks that host their
top-8 of 256 experts as e4m3 rows with one fp32 scale per 128 elements, then combine bf16 result rows
back into a weighted sum per token. Gating is top-8 of N(0,1) logits with softmax weights; data is
synthetic. The reported value is tokens per second for the whole job (sum over ranks).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

Timing: CUDA events on the launching stream around each step (dispatch + combine), L2 flushed
between steps by writing a 512 MiB buffer (outside the timed events), barrier + synchronise on both
sides of the measurement, maximum over ranks. The "e2e" figure repeats the measurement through the
public API with the step's inputs copied from pinned host memory and a result checksum read back
every step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, HIDDEN, EXPERTS, TOPK = 4096, 7168, 256, 8


def reference_arm(args) -> None:
    # The reference is a HIP/CMake C++ library for AMD GPUs (hipcc, ROCm, MPI): it has no Python
    # packaging and cannot be built for sm_100a, and it has no EP dispatch/combine at all.
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is HIP-only (hipcc/ROCm/MPI, no setup.py or pyproject.toml): pip install of "
                          "the reference tree fails and it cannot target sm_100a; it also has no dispatch/combine"}))


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        """Starts nvidia-smi and returns once its first sample has arrived (it needs a moment to
        start, and a short timed region would otherwise end before the first line)."""
        import threading
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        deadline = time.time() + 5.0
        while not self.lines and time.time() < deadline and self.proc.poll() is None:
            time.sleep(0.01)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        out = "".join(self.lines)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=TOKENS)
    ap.add_argument("--layout", default="compact", choices=["compact", "slotted"])
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    args.warmup = max(3, args.warmup)

    import torch
    import torch.distributed as dist

    import rocshmem_b200 as shm
    from rocshmem_b200.ops import collectives as coll
    from rocshmem_b200.ops import moe

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")  # control plane only; the data plane is the symmetric heap
    T = args.tokens
    heap = 6 << 30
    shm.init(heap_size=heap, device=local_rank)
    dev = shm.device()
    d = moe.EpDispatcher(EXPERTS, TOPK, HIDDEN, T, layout=args.layout)
    epr = EXPERTS // world

    g = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(T, HIDDEN, generator=g).to(torch.bfloat16).pin_memory()
    idx_cpu, w_cpu = moe.make_routing(T, EXPERTS, TOPK, 99 + rank)
    idx_host, w_host = idx_cpu.pin_memory(), w_cpu.pin_memory()
    x = x_host.to(dev)
    idx = idx_host.to(dev)
    w = w_host.to(dev)
    y = d.result_buffer()
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    tmax = shm.zeros(4, torch.float64)
    tred = shm.zeros(4, torch.float64)

    def max_over_ranks(values):
        tmax.copy_(torch.tensor(list(values) + [0.0] * (4 - len(values)), dtype=torch.float64))
        torch.cuda.synchronize()
        coll.reduce(tred, tmax, shm.OP_MAX)
        return tred.cpu().tolist()[:len(values)]

    stream = torch.cuda.current_stream()

    def step():
        res = d.dispatch(x, idx, w)
        # "Experts": the combine input has to exist as bf16 rows; the benchmark measures the two
        # collectives, so the rows that arrived are reused as-is (any bf16 content has the same cost).
        d.combine(y, idx, w, T, weighted=True, out=out)
        return res

    # y gets deterministic content once (dequantised rows of a first dispatch) so combine sums real data.
    res = d.dispatch(x, idx, w)
    torch.cuda.synchronize()
    n_rows = res.num_rows()
    y[:n_rows].copy_(moe.fp8_dequantize_1x128(res.recv_x[:n_rows], res.recv_scales[:n_rows]))
    torch.cuda.synchronize()
    shm.barrier_all()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        flush.fill_(1)
        step()
    torch.cuda.synchronize()
    shm.barrier_all()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches_before = d.kernel_launches
    torch.cuda.synchronize()
    shm.barrier_all()
    for i in range(args.steps):
        flush.fill_(i & 0xff)            # L2 flush, outside the timed events
        ev[i][0].record(stream)
        d.dispatch(x, idx, w)
        ev[i][1].record(stream)
        d.combine(y, idx, w, T, weighted=True, out=out)
        ev[i][2].record(stream)
    torch.cuda.synchronize()
    shm.barrier_all()
    phases = d.phase_times_us()
    launches = d.kernel_launches - launches_before
    disp_ms = sum(e[0].elapsed_time(e[1]) for e in ev)
    comb_ms = sum(e[1].elapsed_time(e[2]) for e in ev)
    total_ms, disp_ms, comb_ms = max_over_ranks([disp_ms + comb_ms, disp_ms, comb_ms])
    ms_per_step = total_ms / args.steps

    # ---- end to end through the public API: pinned-host inputs in, checksum out, every step -------------
    h2d_bytes = x_host.numel() * 2 + idx_host.numel() * 4 + w_host.numel() * 4
    checksum_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    # Two sets of device-side inputs: the copy of step i + 1 (on its own stream) overlaps the kernels of step i,
    # as an input pipeline would; every step's copy and every step's result read are inside the timed region.
    copy_stream = torch.cuda.Stream()
    sets = [(x, idx, w), (torch.empty_like(x), torch.empty_like(idx), torch.empty_like(w))]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def issue_copy(i):
        xs, ids, ws = sets[i % 2]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])   # the step that last used this set has finished
            xs.copy_(x_host, non_blocking=True)
            ids.copy_(idx_host, non_blocking=True)
            ws.copy_(w_host, non_blocking=True)
            ready[i % 2].record(copy_stream)

    def e2e_loop(steps):
        issue_copy(0)
        for i in range(steps):
            if i + 1 < steps:
                issue_copy(i + 1)
            xs, ids, ws = sets[i % 2]
            stream.wait_event(ready[i % 2])
            d.dispatch(xs, ids, ws)
            d.combine(y, ids, ws, T, weighted=True, out=out)
            consumed[i % 2].record(stream)
            checksum_host.copy_(out[:, 0].float().sum().reshape(1), non_blocking=True)
            stream.synchronize()                      # the host reads the step's result before the next step

    for e in consumed:
        e.record(stream)
    e2e_loop(max(3, args.warmup))                     # warm-up covers every kernel of the loop, checksum included
    torch.cuda.synchronize()
    shm.barrier_all()
    t0 = time.perf_counter()
    e2e_loop(args.steps)
    torch.cuda.synchronize()
    shm.barrier_all()
    e2e_s = max_over_ranks([time.perf_counter() - t0])[0]
    # The sampler has been running since before the warm-up: it covers both timed regions.
    clocks = sampler.stop() if rank == 0 else None

    # traffic accounting for GB/s (per rank, remote destinations only)
    ranks_of = torch.where(idx_cpu >= 0, idx_cpu // epr, torch.full_like(idx_cpu, -1))
    remote_rows = 0
    for r in range(world):
        if r != rank:
            remote_rows += int((ranks_of == r).any(dim=1).sum())
    disp_bytes = remote_rows * (HIDDEN + HIDDEN // 128 * 4 + 128)
    comb_bytes = remote_rows * HIDDEN * 2
    disp_us = disp_ms / args.steps * 1e3
    comb_us = comb_ms / args.steps * 1e3

    err = shm.get_error()
    if err["count"]:
        raise SystemExit(f"bench: a device-side wait timed out: {err}")

    if rank == 0:
        value = world * T / (ms_per_step * 1e-3)
        line = {
            "metric": "ep_dispatch_combine_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8-e4m3 dispatch / bf16 combine",
            "data": "synthetic", "impl": "ours",
            "config": {"model": "DeepEP-style MoE dispatch+combine (DeepSeek-V3-like)", "experts": EXPERTS,
                       "experts_per_rank": epr, "top_k": TOPK, "hidden": HIDDEN, "tokens_per_rank": T,
                       "global_batch": world * T, "seq_len": 1, "parallelism": f"ep{world}",
                       "layout": args.layout, "dynamic_handout": bool(d.dynamic),
                       "l2": "flushed between steps (512 MiB write)",
                       "dispatch": "fp8 e4m3 + fp32 scale per 128", "combine": "bf16 weighted sum"},
            "clocks": clocks,
            "e2e": {"value": world * T * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "extra": {"dispatch_us": disp_us, "combine_us": comb_us,
                      "dispatch_remote_gbs_per_rank": disp_bytes / (disp_us * 1e-6) / 1e9 if remote_rows else 0.0,
                      "combine_remote_gbs_per_rank": comb_bytes / (comb_us * 1e-6) / 1e9 if remote_rows else 0.0,
                      "remote_rows_rank0": remote_rows, "recv_rows_rank0": n_rows,
                      "device_phase_us_last_step": phases,
                      "nvlink_roofline_frac_dispatch": (disp_bytes / 770e9) / (disp_us * 1e-6) if remote_rows else None,
                      "nvlink_roofline_frac_combine": (comb_bytes / 770e9) / (comb_us * 1e-6) if remote_rows else None},
        }
        print(json.dumps(line))
    shm.finalize()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
