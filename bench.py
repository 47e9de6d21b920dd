#!/usr/bin/env python
"""Headline benchmark: DeepEP-style expert-parallel dispatch + combine on N GPUs of one node.

One step = for every rank, dispatch 4096 bf16 tokens (hidden 7168) to the ranks that host their
top-8 of 256 experts as e4m3 rows with one fp32 scale per 128 elements, then combine bf16 result rows
back into a weighted sum per token. Gating is top-8 of N(0,1) logits with softmax weights; data is
synthetic. The reported value is tokens per second for the whole job (sum over ranks).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

A step is R dispatch+combine pairs (R is chosen so that a step lasts about 3 ms and is reported as
``pairs_per_step``). Timing: CUDA events on the launching stream around each pair, L2 flushed before every
pair by writing a 512 MiB buffer (outside the timed events), barrier + synchronise on both sides of the
measurement, maximum over ranks. One pair is checked on every rank before anything is timed (``verified``).
The same workload is then run over NCCL all-to-all (``baseline``; ``vs_baseline`` is ours / NCCL). The
"e2e" figure repeats the measurement through the public API with the step's inputs copied from pinned
host memory and a result checksum read back every step. A short run of the low-latency kernels (128 tokens
per rank) follows and is reported under ``extra`` (``--no-ll-extra`` leaves it out), and with two or more GPUs a
short comparison of the library collectives with NCCL (``--no-coll-extra``).
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


def h2d_ceiling_gbs(torch, host, dev, reps: int = 5) -> float:
    """Plain pinned-host -> device copy rate of this rank (GB/s), the ceiling of the end-to-end figure."""
    dst = torch.empty_like(host, device=dev)
    for _ in range(2):
        dst.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        dst.copy_(host, non_blocking=True)
    b.record()
    torch.cuda.synchronize()
    return host.numel() * host.element_size() * reps / (a.elapsed_time(b) * 1e-3) / 1e9


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=TOKENS)
    ap.add_argument("--layout", default="compact", choices=["compact", "slotted"])
    ap.add_argument("--low-latency", action="store_true", help="low-latency kernels (use with --tokens 128)")
    ap.add_argument("--repeats", type=int, default=0,
                    help="dispatch+combine pairs per step (0: as many as make a step last about 3 ms)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL all-to-all form of the workload")
    ap.add_argument("--no-ll-extra", action="store_true",
                    help="skip the short low-latency measurement (128 tokens per rank) reported under extra")
    ap.add_argument("--no-coll-extra", action="store_true",
                    help="skip the short collective measurements (allreduce, all-gather, all-to-all, broadcast against "
                         "NCCL) reported under extra when there are two or more GPUs")
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
    from rocshmem_b200.utils import numa

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    # Pinned input buffers on the GPU's own NUMA node: otherwise the ranks' host-to-device copies share one
    # socket's memory and the inter-socket link.
    numa_info = numa.bind_to_device_node(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        import socket
        with socket.socket() as sock:                # single process: any free port will do
            sock.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(sock.getsockname()[1])
    # gloo is the control plane of the symmetric heap's bootstrap; NCCL carries only the baseline's all-to-all.
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", local_rank))
    T = args.tokens
    heap = 6 << 30
    shm.init(heap_size=heap, device=local_rank)
    dev = shm.device()
    d = moe.EpDispatcher(EXPERTS, TOPK, HIDDEN, T, layout=args.layout, low_latency=args.low_latency)
    epr = EXPERTS // world

    g = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(T, HIDDEN, generator=g).to(torch.bfloat16).pin_memory()
    routes = [moe.make_routing(T, EXPERTS, TOPK, 99 + r) for r in range(world)]
    idx_cpu, w_cpu = routes[rank]
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

    # y gets deterministic content once (dequantised rows of a first dispatch) so combine sums real data.
    res = d.dispatch(x, idx, w)
    torch.cuda.synchronize()
    info = res.recv_info.cpu().tolist()
    n_rows = info[0]
    for s in range(world):
        first, count = info[1 + s], info[1 + world + s]
        if count:
            y[first:first + count].copy_(moe.fp8_dequantize_1x128(res.recv_x[first:first + count],
                                                                  res.recv_scales[first:first + count]))
    torch.cuda.synchronize()
    shm.barrier_all()

    # ---- correctness of one step, on every rank, before anything is timed ---------------------------------------
    # Bookkeeping against the reference routing of all ranks (their gating is rebuilt from the seeds), and the
    # combine output against the fp32 weighted sum of the de-quantised rows (the gate weights sum to one, so
    # that sum is the de-quantised token itself).
    want_rows = moe.ref_dispatch([r[0] for r in routes], world, EXPERTS)[rank]
    bad = 0.0
    if n_rows != len(want_rows):
        bad = 1.0
    meta = res.recv_meta.cpu()
    for s in range(world):
        first, count = info[1 + s], info[1 + world + s]
        toks = sorted(meta[first:first + count, 16].tolist())
        if toks != [t for ss, t in want_rows if ss == s]:
            bad = 1.0
    d.combine(y, idx, w, T, weighted=True, out=out)
    torch.cuda.synchronize()
    xf = x.float()
    if (out.float() - xf).abs().max().item() > 0.08 * xf.abs().max().item() + 2e-2:
        bad = 1.0
    del xf
    verified = max_over_ranks([bad])[0] == 0.0
    shm.barrier_all()

    def pair(events=None):
        if events:
            events[0].record(stream)
        d.dispatch(x, idx, w)
        if events:
            events[1].record(stream)
        d.combine(y, idx, w, T, weighted=True, out=out)
        if events:
            events[2].record(stream)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        flush.fill_(1)
        pair()
    torch.cuda.synchronize()
    # Pairs per step: enough for a step of about 3 ms, so that the timed region is long enough for the clock
    # samples to mean something. Every rank derives the same number from the maximum over ranks.
    if args.repeats > 0:
        R = args.repeats
    else:
        probe = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        flush.fill_(2)
        pair(probe)
        torch.cuda.synchronize()
        pair_ms = max_over_ranks([probe[0].elapsed_time(probe[2])])[0]
        R = int(max(1, min(64, round(3.0 / max(pair_ms, 1e-3)))))
    shm.barrier_all()
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(R)] for _ in range(args.steps)]
    launches_before = d.kernel_launches
    torch.cuda.synchronize()
    shm.barrier_all()
    for i in range(args.steps):
        for r in range(R):
            flush.fill_((i + r) & 0xff)      # L2 flush, outside the timed events
            pair(ev[i][r])
    torch.cuda.synchronize()
    shm.barrier_all()
    phases = d.phase_times_us()
    launches = d.kernel_launches - launches_before
    disp_ms = sum(e[0].elapsed_time(e[1]) for step in ev for e in step)
    comb_ms = sum(e[1].elapsed_time(e[2]) for step in ev for e in step)
    total_ms, disp_ms, comb_ms = max_over_ranks([disp_ms + comb_ms, disp_ms, comb_ms])
    ms_per_step = total_ms / args.steps
    pairs = args.steps * R

    # ---- the same workload over NCCL all-to-all (the library baseline), same tensors, same timing rules -----------
    base = None
    if not args.no_baseline:
        from rocshmem_b200.baselines.ep import NcclEpDispatcher
        nd = NcclEpDispatcher(EXPERTS, TOPK, HIDDEN)
        nres = nd.dispatch(x, idx, w)
        ny = moe.fp8_dequantize_1x128(nres.recv_x, nres.recv_scales) if nres.recv_x.shape[0] else \
            torch.empty((0, HIDDEN), dtype=torch.bfloat16, device=dev)
        nout = nd.combine(ny, idx, w, T)
        base_ok = (nout.float() - x.float()).abs().max().item() <= 0.08 * x.float().abs().max().item() + 2e-2
        for _ in range(3):
            flush.fill_(3)
            nd.dispatch(x, idx, w)
            nd.combine(ny, idx, w, T)
        torch.cuda.synchronize()
        dist.barrier()
        nsteps = max(3, min(pairs, 40))
        nev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(nsteps)]
        for i in range(nsteps):
            flush.fill_(i & 0xff)
            nev[i][0].record(stream)
            nd.dispatch(x, idx, w)
            nev[i][1].record(stream)
            nd.combine(ny, idx, w, T)
            nev[i][2].record(stream)
        torch.cuda.synchronize()
        dist.barrier()
        bd = sum(e[0].elapsed_time(e[1]) for e in nev)
        bc = sum(e[1].elapsed_time(e[2]) for e in nev)
        btot, bd, bc = max_over_ranks([bd + bc, bd, bc])
        base = {"impl": "NCCL all_to_all_single (torch.distributed) + torch kernels", "pairs_timed": nsteps,
                "ms_per_pair": btot / nsteps, "dispatch_us": bd / nsteps * 1e3, "combine_us": bc / nsteps * 1e3,
                "value": world * T / (btot / nsteps * 1e-3), "verified": bool(base_ok)}
        del nd, nres, ny, nout

    # ---- end to end through the public API: pinned-host inputs in, result checksum out, every step ----------------
    h2d_bytes = x_host.numel() * 2 + idx_host.numel() * 4 + w_host.numel() * 4
    h2d_gbs = max_over_ranks([-h2d_ceiling_gbs(torch, x_host, dev)])[0] * -1.0   # slowest rank
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
    e2e_steps = max(args.steps, min(200, pairs))
    e2e_loop(max(3, args.warmup))                     # warm-up covers every kernel of the loop, checksum included
    torch.cuda.synchronize()
    shm.barrier_all()
    t0 = time.perf_counter()
    e2e_loop(e2e_steps)
    torch.cuda.synchronize()
    shm.barrier_all()
    e2e_s = max_over_ranks([time.perf_counter() - t0])[0]
    # The sampler has been running since before the warm-up: it covers both timed regions.
    clocks = sampler.stop() if rank == 0 else None

    # ---- low-latency kernels, 128 tokens per rank: a short side measurement, reported under "extra" -----------------
    # It runs after everything the headline needs has been measured; whatever goes wrong in it is reported in its
    # own entry and leaves the numbers above alone.
    err = shm.get_error()          # the record of everything measured so far
    dynamic_handout = bool(d.dynamic)
    ll_extra = None
    if not err["count"] and not args.low_latency and not args.no_ll_extra:
        try:
            TL = min(128, T)
            d.destroy()                 # one dispatcher at a time, as everywhere else; its numbers are all in hand
            dl = moe.EpDispatcher(EXPERTS, TOPK, HIDDEN, TL, low_latency=True)
            xl, il, wl = x[:TL].clone(), idx[:TL].clone(), w[:TL].clone()
            yl = dl.result_buffer()
            outl = torch.empty((TL, HIDDEN), dtype=torch.bfloat16, device=dev)
            rl = dl.dispatch(xl, il, wl)
            torch.cuda.synchronize()
            infol = rl.recv_info.cpu().tolist()
            for s in range(world):
                first, count = infol[1 + s], infol[1 + world + s]
                if count:
                    yl[first:first + count].copy_(moe.fp8_dequantize_1x128(rl.recv_x[first:first + count],
                                                                           rl.recv_scales[first:first + count]))
            torch.cuda.synchronize()
            shm.barrier_all()
            dl.combine(yl, il, wl, TL, weighted=True, out=outl)
            torch.cuda.synchronize()
            xlf = xl.float()
            ll_bad = float((outl.float() - xlf).abs().max().item() > 0.08 * xlf.abs().max().item() + 2e-2)
            for _ in range(5):
                flush.fill_(5)
                dl.dispatch(xl, il, wl)
                dl.combine(yl, il, wl, TL, weighted=True, out=outl)
            torch.cuda.synchronize()
            shm.barrier_all()
            n_ll = 40
            lev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_ll)]
            for i in range(n_ll):
                flush.fill_(i & 0xff)
                lev[i][0].record(stream)
                dl.dispatch(xl, il, wl)
                lev[i][1].record(stream)
                dl.combine(yl, il, wl, TL, weighted=True, out=outl)
                lev[i][2].record(stream)
            torch.cuda.synchronize()
            shm.barrier_all()
            ld = sum(e[0].elapsed_time(e[1]) for e in lev) / n_ll * 1e3
            lc = sum(e[1].elapsed_time(e[2]) for e in lev) / n_ll * 1e3
            ld, lc, ll_bad = max_over_ranks([ld, lc, ll_bad])
            ll_err = shm.get_error()
            dl.destroy()
            if ll_err["count"]:
                shm.clear_error()
                ll_extra = {"error": f"a device-side wait timed out: {ll_err}"}
            else:
                ll_extra = {"tokens_per_rank": TL, "pairs_timed": n_ll, "dispatch_us": ld, "combine_us": lc,
                            "verified": ll_bad == 0.0, "layout": "slotted"}
        except Exception as e:      # noqa: BLE001 - a side measurement must not cost the headline
            ll_extra = {"error": f"{type(e).__name__}: {e}"}

    # ---- library collectives against NCCL on the same GPUs: a short side measurement, reported under "extra" --------
    # Back-to-back launches (no L2 flush: the large messages exceed the L2, the small ones measure latency), three
    # warm-ups, CUDA events, maximum over ranks; the same rules for both sides. Guarded like the measurement above.
    coll_extra = None
    if world >= 2 and not err["count"] and not args.no_coll_extra and not (ll_extra and "error" in ll_extra):
        try:
            big = 64 << 20                                   # bytes
            csrc = shm.zeros(big // 2, torch.bfloat16)
            cdst = shm.zeros(big // 2, torch.bfloat16)
            nsrc = torch.empty(big // 2, dtype=torch.bfloat16, device=dev)
            ndst = torch.empty(big // 2, dtype=torch.bfloat16, device=dev)
            csrc.normal_()
            nsrc.copy_(csrc)
            ndst.zero_()
            torch.cuda.synchronize()
            shm.barrier_all()

            def timed(fn, iters):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                shm.barrier_all()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(iters):
                    fn()
                b.record(stream)
                torch.cuda.synchronize()
                return max_over_ranks([a.elapsed_time(b) * 1e3 / iters])[0]

            rows = []
            busf = 2.0 * (world - 1) / world
            for nbytes in (1 << 10, 256 << 10, 64 << 20):
                n, iters = nbytes // 2, (50 if nbytes <= (1 << 20) else 8)
                ours = timed(lambda: coll.allreduce_async(cdst[:n], csrc[:n], shm.OP_SUM), iters)

                theirs = timed(lambda: dist.all_reduce(ndst[:n]), iters)      # in place, NCCL's own calling form
                rows.append({"op": "allreduce", "bytes": nbytes, "dtype": "bf16", "us": ours, "nccl_us": theirs,
                             "busbw_gbs": busf * nbytes / ours / 1e3, "nccl_busbw_gbs": busf * nbytes / theirs / 1e3})
            # the allreduce is checked once against an fp32 sum gathered over NCCL
            n_chk = 4096
            coll.allreduce_async(cdst[:n_chk], csrc[:n_chk], shm.OP_SUM)
            parts = [torch.empty(n_chk, dtype=torch.bfloat16, device=dev) for _ in range(world)]
            dist.all_gather(parts, csrc[:n_chk].clone())
            torch.cuda.synchronize()
            want = sum(p.float() for p in parts)
            coll_bad = float((cdst[:n_chk].float() - want).abs().max().item() > 3e-2 * max(1.0, want.abs().max().item()))
            per = (big // world) // 2 // 8 * 8                # elements per peer, 16-byte multiples
            for name, ours_fn, nccl_fn, moved in (
                ("fcollect", lambda: coll.fcollect_async(cdst[:per * world], csrc[:per]),
                 lambda: dist.all_gather_into_tensor(ndst[:per * world], nsrc[:per]), per * 2 * (world - 1)),
                ("alltoall", lambda: coll.alltoall_async(cdst[:per * world], csrc[:per * world]),
                 lambda: dist.all_to_all_single(ndst[:per * world], nsrc[:per * world]), per * 2 * (world - 1)),
                ("broadcast", lambda: coll.broadcast_async(cdst, csrc, 0), lambda: dist.broadcast(nsrc, 0), big),
            ):
                ours = timed(ours_fn, 8)
                theirs = timed(nccl_fn, 8)
                rows.append({"op": name, "bytes_per_peer": per * 2 if name != "broadcast" else big, "us": ours,
                             "nccl_us": theirs, "gbs": moved / ours / 1e3, "nccl_gbs": moved / theirs / 1e3})
            coll_bad = max_over_ranks([coll_bad])[0]
            coll_err = shm.get_error()
            if coll_err["count"]:
                shm.clear_error()
                coll_extra = {"error": f"a device-side wait timed out: {coll_err}"}
            else:
                coll_extra = {"rows": rows, "allreduce_verified": coll_bad == 0.0, "nvls": bool(shm.nvls_available()),
                              "note": "back-to-back launches, 3 warm-ups, CUDA events, max over ranks; GB/s of the copy "
                                      "collectives = bytes entering one rank / time"}
        except Exception as e:      # noqa: BLE001 - a side measurement must not cost the headline
            coll_extra = {"error": f"{type(e).__name__}: {e}"}

    # traffic accounting for GB/s (per rank, remote destinations only)
    ranks_of = torch.where(idx_cpu >= 0, idx_cpu // epr, torch.full_like(idx_cpu, -1))
    remote_rows = 0
    for r in range(world):
        if r != rank:
            remote_rows += int((ranks_of == r).any(dim=1).sum())
    disp_bytes = remote_rows * (HIDDEN + HIDDEN // 128 * 4 + 128)
    comb_bytes = remote_rows * HIDDEN * 2
    disp_us = disp_ms / pairs * 1e3
    comb_us = comb_ms / pairs * 1e3

    if err["count"]:
        raise SystemExit(f"bench: a device-side wait timed out: {err}")

    if rank == 0:
        value = world * T * R / (ms_per_step * 1e-3)

        def frac(nbytes, us, gbs):
            return (nbytes / (gbs * 1e9)) / (us * 1e-6) if remote_rows else None

        line = {
            "metric": "ep_dispatch_combine_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak",
            # No published number exists for the reference; the ratio is against the NCCL form measured above.
            "vs_baseline": (value / base["value"]) if base else None,
            "dtype": "fp8-e4m3 dispatch / bf16 combine",
            "data": "synthetic", "impl": "ours", "verified": bool(verified),
            "config": {"model": "DeepEP-style MoE dispatch+combine (DeepSeek-V3-like)", "experts": EXPERTS,
                       "experts_per_rank": epr, "top_k": TOPK, "hidden": HIDDEN, "tokens_per_rank": T,
                       "pairs_per_step": R, "global_batch": world * T * R, "seq_len": 1, "parallelism": f"ep{world}",
                       "layout": "slotted" if args.low_latency else args.layout, "low_latency": bool(args.low_latency),
                       "dynamic_handout": dynamic_handout,
                       "l2": "flushed before every dispatch+combine pair (512 MiB write, outside the timed events)",
                       "dispatch": "fp8 e4m3 + fp32 scale per 128", "combine": "bf16 weighted sum"},
            "clocks": clocks,
            "e2e": {"value": world * T * e2e_steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4, "d2h": "fp32 checksum of the step's output (one scalar, like a loss)",
                    "steps": e2e_steps, "pairs_per_step": 1,
                    "h2d_ceiling_gbs_slowest_rank": h2d_gbs,
                    "h2d_ceiling_tokens_per_s": world * T * (h2d_gbs * 1e9 / h2d_bytes), "numa": numa_info},
            "gpu_launches": launches,
            "baseline": base,
            "extra": {"dispatch_us": disp_us, "combine_us": comb_us,
                      "dispatch_remote_gbs_per_rank": disp_bytes / (disp_us * 1e-6) / 1e9 if remote_rows else 0.0,
                      "combine_remote_gbs_per_rank": comb_bytes / (comb_us * 1e-6) / 1e9 if remote_rows else 0.0,
                      "remote_rows_rank0": remote_rows, "recv_rows_rank0": n_rows,
                      "device_phase_us_last_step": phases,
                      "low_latency_128_tokens": ll_extra,
                      "collectives_vs_nccl": coll_extra,
                      "nvlink_roofline_frac_dispatch": {"of_measured_770": frac(disp_bytes, disp_us, 770),
                                                        "of_link_rate_900": frac(disp_bytes, disp_us, 900)},
                      "nvlink_roofline_frac_combine": {"of_measured_770": frac(comb_bytes, comb_us, 770),
                                                       "of_link_rate_900": frac(comb_bytes, comb_us, 900)}},
        }
        print(json.dumps(line))
    shm.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
