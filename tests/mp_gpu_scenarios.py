"""Multi-process GPU scenarios: one PE per process and per GPU, device API from user kernels and
the library's stream-ordered collectives over real NVLink peer mappings."""
import os

import torch

import rocshmem_b200 as shm
from rocshmem_b200 import _native
from rocshmem_b200.ops import collectives as coll

RANK = int(os.environ["RANK"])
WORLD = int(os.environ["WORLD_SIZE"])


def _init(heap="512M", **kw):
    shm.init(heap_size=heap, backend="cuda", ROCSHMEM_WAIT_TIMEOUT_MS=5000, **kw)
    assert shm.is_cuda() and shm.n_pes() == WORLD and shm.my_pe() == RANK
    return _native.load_test_kernels()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ok():
    torch.cuda.synchronize()
    err = shm.get_error()
    assert err["count"] == 0, err


def gpu_device_suite():
    k = _init()
    me, n = RANK, WORLD
    dev = shm.device()
    # put / get, all scopes
    for op in range(4):
        for scope in range(3):
            nbytes = 1 << 20
            src = shm.zeros(nbytes, torch.uint8)
            dst = shm.zeros(nbytes, torch.uint8)
            g = torch.Generator().manual_seed(100 + me)
            src.copy_(torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).to(dev))
            torch.cuda.synchronize()
            shm.barrier_all()
            k.rma(op, scope, dst.data_ptr(), src.data_ptr(), nbytes, 1, 1, 256 if scope else 64, _stream())
            _ok()
            origin = (me - 1) % n if op < 2 else (me + 1) % n
            g = torch.Generator().manual_seed(100 + origin)
            assert torch.equal(dst.cpu(), torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8)), (op, scope)
            shm.free(dst)
            shm.free(src)
    # atomics from every PE onto PE 0
    target = shm.zeros(1, torch.int64)
    ret = shm.zeros(128, torch.int64)
    k.amo(0, target.data_ptr(), ret.data_ptr(), 10, 2, 64, _stream())
    _ok()
    shm.barrier_all()
    if me == 0:
        assert int(target.cpu()[0]) == 2 * n * 128 * 10
    # signals, ping-pong, ping-all, barrier stress
    nbytes = 8192
    src = shm.zeros(nbytes, torch.uint8)
    dst = shm.zeros(nbytes, torch.uint8)
    sig = shm.zeros(1, torch.int64)
    fetched = shm.zeros(2, torch.int64)
    src.fill_(ord("0") + me)
    torch.cuda.synchronize()
    shm.barrier_all()
    k.signal(2, 0, dst.data_ptr(), src.data_ptr(), nbytes, sig.data_ptr(), 7, 7, fetched.data_ptr(), 64, _stream())
    _ok()
    assert fetched.cpu().tolist() == [7, 0] and torch.all(dst.cpu() == ord("0") + (me - 1) % n)
    flag = shm.zeros(1, torch.int32)
    ns = shm.zeros(1, torch.int64)
    k.pingpong(flag.data_ptr(), 1000, ns.data_ptr(), _stream())
    _ok()
    if me == 0:
        print(f"ping-pong round trip: {int(ns.cpu()[0]) / 1000:.0f} ns")
    slots = shm.zeros(n, torch.int64)
    result = shm.zeros(8, torch.int64)
    k.pingall(slots.data_ptr(), result.data_ptr(), _stream())
    _ok()
    assert slots.cpu().tolist() == [p + 1 for p in range(n)]
    errors = shm.zeros(1, torch.int32)
    k.barrier_stress(slots.data_ptr(), 500, errors.data_ptr(), 64, _stream())
    _ok()
    assert int(errors.cpu()[0]) == 0
    # block collectives from user kernels
    x = shm.zeros(5000, torch.float32)
    y = shm.zeros(5000, torch.float32)
    rc = shm.zeros(1, torch.int32)
    x.copy_((torch.arange(5000, dtype=torch.float32) * (me + 1)).to(dev))
    torch.cuda.synchronize()
    shm.barrier_all()
    k.coll(3, "float32", shm.team_world().handle, y.data_ptr(), x.data_ptr(), 5000, 0, 3, rc.data_ptr(), 512, _stream())
    _ok()
    assert torch.allclose(y.cpu(), torch.arange(5000, dtype=torch.float32) * (n * (n + 1) // 2))
    shm.barrier_all()
    before = torch.cuda.current_device()
    shm.finalize()
    # finalize leaves the caller's current device alone (it clears the modules' state on the heap's device only)
    assert torch.cuda.current_device() == before == dev.index, (before, torch.cuda.current_device(), dev)
    assert torch.ones(4, device="cuda").device.index == dev.index


def gpu_library_collectives():
    _init("2G")
    me, n = RANK, WORLD
    dev = shm.device()
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.float64):
        for nelem in (1, 1000, 65536 + 8, 3 << 20):
            src = shm.zeros(nelem, dtype)
            dst = shm.zeros(nelem, dtype)
            g = torch.Generator().manual_seed(9 + me)
            ins = []
            for p in range(n):
                gp = torch.Generator().manual_seed(9 + p)
                if dtype.is_floating_point:
                    ins.append(torch.randn(nelem, generator=gp, dtype=torch.float32).to(dtype))
                else:
                    ins.append(torch.randint(-1000, 1000, (nelem,), generator=gp, dtype=torch.int64).to(dtype))
            src.copy_(ins[me].to(dev))
            torch.cuda.synchronize()
            shm.barrier_all()
            ref = torch.stack([i.to(torch.float64) for i in ins]).sum(0)
            algos = [shm.ALLREDUCE_ONE_SHOT, shm.ALLREDUCE_TWO_SHOT, shm.ALLREDUCE_AUTO]
            if shm.nvls_available() and dtype in (torch.float32, torch.bfloat16, torch.float16) and nelem % 8 == 0:
                algos.append(shm.ALLREDUCE_NVLS)
            for algo in algos:
                dst.zero_()
                coll.allreduce_async(dst, src, shm.OP_SUM, algo=algo)
                _ok()
                tol = {torch.bfloat16: 3e-2, torch.float16: 5e-3}.get(dtype, 1e-5)
                assert torch.allclose(dst.cpu().to(torch.float64), ref, rtol=tol, atol=tol * n), (dtype, nelem, algo)
            coll.allreduce_async(dst, src, shm.OP_MAX, algo=shm.ALLREDUCE_TWO_SHOT)
            _ok()
            refmax = torch.stack([i.to(torch.float64) for i in ins]).max(0).values
            assert torch.allclose(dst.cpu().to(torch.float64), refmax), (dtype, nelem, "max")
            shm.barrier_all()
            shm.free(dst)
            shm.free(src)
    nbytes = 5 << 20
    src = shm.zeros(nbytes * n, torch.uint8)
    dst = shm.zeros(nbytes * n, torch.uint8)
    src.fill_(me + 1)
    torch.cuda.synchronize()
    shm.barrier_all()
    coll.fcollect_async(dst, src[:nbytes])
    _ok()
    got = dst.cpu().view(n, nbytes)
    assert all(torch.all(got[p] == p + 1) for p in range(n))
    for p in range(n):
        src.view(n, nbytes)[p].fill_(10 * me + p)
    torch.cuda.synchronize()
    coll.alltoall_async(dst, src)
    _ok()
    got = dst.cpu().view(n, nbytes)
    assert all(torch.all(got[p] == 10 * p + me) for p in range(n))
    dst.zero_()
    torch.cuda.synchronize()
    coll.broadcast_async(dst[:nbytes], src[:nbytes], n - 1)
    _ok()
    if me != n - 1:
        assert torch.all(dst.cpu()[:nbytes] == 10 * (n - 1))
    shm.barrier_all()
    print(f"nvls={shm.nvls_available()}")
    shm.finalize()


def gpu_team_nvls():
    """Split teams with a multicast mapping of their own: two disjoint halves and the even / odd PEs exist at the
    same time (every PE is a member of two of them), run the switch-side allreduce, all-gather and broadcast,
    are destroyed and split again with other members, and one team is still alive at finalize."""
    os.environ["ROCSHMEM_BCAST_NVLS"] = "1"
    os.environ["ROCSHMEM_FCOLLECT_NVLS"] = "1"
    _init("1G")
    me, n = RANK, WORLD
    dev = shm.device()
    world = shm.team_world()
    nelem, nbytes = 3 << 20, 5 << 20
    src = shm.zeros(nelem, torch.float32)
    dst = shm.zeros(nelem, torch.float32)
    bsrc = shm.zeros(nelem, torch.bfloat16)
    bdst = shm.zeros(nelem, torch.bfloat16)
    gsrc = shm.zeros(nbytes, torch.uint8)
    gdst = shm.zeros(nbytes * n, torch.uint8)
    ins = [torch.randn(nelem, generator=torch.Generator().manual_seed(40 + p)) for p in range(n)]
    src.copy_(ins[me].to(dev))
    bsrc.copy_(ins[me].to(torch.bfloat16).to(dev))
    gsrc.fill_(me + 1)
    torch.cuda.synchronize()
    shm.barrier_all()

    def check(team, members, tag):
        if me not in members:
            return
        m = len(members)
        assert team.valid and team.n_pes() == m and team.my_pe() == members.index(me), tag
        assert team.has_nvls() == (shm.nvls_available() and m >= 2), (tag, team.has_nvls())
        ref = torch.stack([ins[p].double() for p in members]).sum(0)
        bref = torch.stack([ins[p].to(torch.bfloat16).double() for p in members]).sum(0)
        for algo in (shm.ALLREDUCE_AUTO, shm.ALLREDUCE_NVLS, shm.ALLREDUCE_TWO_SHOT):
            dst.zero_()
            bdst.zero_()
            coll.allreduce_async(dst, src, shm.OP_SUM, team=team, algo=algo)
            coll.allreduce_async(bdst, bsrc, shm.OP_SUM, team=team, algo=algo)
            _ok()
            assert torch.allclose(dst.cpu().double(), ref, rtol=1e-5, atol=1e-5 * m), (tag, algo)
            assert torch.allclose(bdst.cpu().double(), bref, rtol=3e-2, atol=3e-2 * m), (tag, algo, "bf16")
        gdst.zero_()
        coll.fcollect_async(gdst[:nbytes * m], gsrc, team=team)
        _ok()
        got = gdst.cpu()[:nbytes * m].view(m, nbytes)
        assert all(torch.all(got[i] == members[i] + 1) for i in range(m)), tag
        gdst.zero_()
        torch.cuda.synchronize()
        team.sync()
        coll.broadcast_async(gdst[:nbytes], gsrc, m - 1, team=team)
        _ok()
        if me != members[-1]:
            assert torch.all(gdst.cpu()[:nbytes] == members[-1] + 1), tag
        team.sync()

    half = max(1, n // 2)
    lower, upper = list(range(half)), list(range(half, n))
    evens, odds = list(range(0, n, 2)), list(range(1, n, 2))
    t_lo = world.split_strided(0, 1, half)
    t_hi = world.split_strided(half, 1, n - half)
    t_ev = world.split_strided(0, 2, len(evens))
    t_od = world.split_strided(1, 2, len(odds)) if odds else None
    for rep in range(2):
        check(t_lo, lower, "lower")
        check(t_hi, upper, "upper")
        check(t_ev, evens, "even")
        if odds:
            check(t_od, odds, "odd")
    check(world, list(range(n)), "world")
    for t in (t_lo, t_hi, t_ev, t_od):
        if t is not None and t.valid:
            t.destroy()
    shm.barrier_all()
    # the freed slots are taken by teams with other members
    if n >= 3:
        rest = list(range(1, n))
        t_rest = world.split_strided(1, 1, n - 1)
        check(t_rest, rest, "all but PE 0")
        t_ends = world.split_strided(0, n - 1, 2)
        check(t_ends, [0, n - 1], "first and last")
    _ok()
    shm.barrier_all()
    print(f"nvls={shm.nvls_available()}")
    shm.finalize()    # with teams (and their mappings) still alive


C_BCAST, C_FCOLLECT, C_ALLTOALL, C_SUM = 0, 1, 2, 3


def gpu_proxied_collectives():
    """Two processes, one GPU each: block-level reduce, fcollect and broadcast of a kernel run through the proxy."""
    k = _init("64M", ROCSHMEM_USE_PROXY=1, ROCSHMEM_PROXY_COLLECTIVES=1, ROCSHMEM_ENABLE_NVLS=0)
    rank, world = RANK, WORLD
    n = 1024
    src = shm.zeros(n * world, torch.float32)
    dst = shm.zeros(n * world, torch.float32)
    rc = shm.zeros(4, torch.int32)
    src.copy_((torch.arange(n * world) + 1000 * rank).float().cuda())
    torch.cuda.synchronize()
    shm.barrier_all()
    side = torch.cuda.Stream()
    team = shm.team_world().handle

    def run(op, count, root=0):
        with torch.cuda.stream(side):
            k.coll(op, "float32", team, dst.data_ptr(), src.data_ptr(), count, root, 1, rc.data_ptr(), 128, side.cuda_stream)
        torch.cuda.synchronize()
        assert shm.get_error()["count"] == 0, shm.get_error()

    run(C_SUM, n)
    want = torch.arange(n).float() * world + 1000.0 * sum(range(world))
    assert torch.equal(dst.cpu()[:n], want)
    run(C_FCOLLECT, n)
    got = dst.cpu().view(world, n)
    assert all(torch.equal(got[r], torch.arange(n).float() + 1000 * r) for r in range(world))
    dst.zero_()
    torch.cuda.synchronize()
    shm.barrier_all()
    run(C_BCAST, n, root=world - 1)
    if rank != world - 1:
        assert torch.equal(dst.cpu()[:n], torch.arange(n).float() + 1000 * (world - 1))
    shm.barrier_all()
    shm.finalize()
    print(f"rank {rank}: proxied collectives ok")


def gpu_moe():
    """Dispatch + combine across real GPUs: identity experts return the token, rank-constant rows
    give exact sums, routing bookkeeping matches a CPU reference."""
    from rocshmem_b200.ops import moe
    _init("4G")
    me, n = RANK, WORLD
    dev = shm.device()
    for layout, (T, H, E, K) in (("compact", (1000, 7168, 8 * n, 8 if n >= 2 else 4)), ("slotted", (128, 2048, 4 * n, 4))):
        K = min(K, E)
        d = moe.EpDispatcher(E, K, H, T, layout=layout)
        epr = E // n
        for rep in range(3):
            g = torch.Generator().manual_seed(50 * rep + me)
            x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
            routes = [moe.make_routing(T, E, K, 1000 * rep + p) for p in range(n)]
            idx, w = routes[me][0].to(dev), routes[me][1].to(dev)
            res = d.dispatch(x, idx, w)
            _ok()
            want_rows = moe.ref_dispatch([r[0] for r in routes], n, E)[me]
            info = res.recv_info.cpu().tolist()
            assert info[0] == len(want_rows), (info[0], len(want_rows))
            meta = res.recv_meta.cpu()
            pos = 0
            for s in range(n):
                first, count = info[1 + s], info[1 + n + s]
                src = [t for ss, t in want_rows if ss == s]
                assert count == len(src) and first == (s * T if layout == "slotted" else pos)
                pos += count
                assert meta[first:first + count, 16].tolist() == src
                assert meta[first:first + count, 17].tolist() == [s] * count
            y = d.result_buffer()
            for s in range(n):
                first, count = info[1 + s], info[1 + n + s]
                if count:
                    y[first:first + count].copy_(moe.fp8_dequantize_1x128(res.recv_x[first:first + count],
                                                                          res.recv_scales[first:first + count]))
            out = d.combine(y, idx, w, T, weighted=True)
            _ok()
            assert (out.float() - x.float()).abs().max().item() <= 0.08 * x.float().abs().max().item() + 2e-2
            y.fill_(float(me + 1))
            out = d.combine(y, idx, w, T, weighted=False)
            _ok()
            ranks = torch.where(routes[me][0] >= 0, routes[me][0] // epr, torch.full_like(routes[me][0], -1))
            want = torch.zeros(T)
            for r in range(n):
                want += (ranks == r).any(dim=1).float() * (r + 1)
            assert torch.equal(out[:, 0].float().cpu(), want) and torch.equal(out[:, -1].float().cpu(), want)
            shm.barrier_all()
    shm.finalize()


def gpu_tp_fused():
    """all-gather -> GEMM and GEMM -> reduce-scatter against a torch reference built from every rank's
    (seeded) inputs."""
    from rocshmem_b200.ops import gemm
    _init("2G")
    me, n = RANK, WORLD
    dev = shm.device()
    for m_shard, K, N in ((128, 512, 256), (256, 1024, 1000 // 8 * 8), (384, 2048, 1792)):
        tp = gemm.TensorParallelLinear(m_shard)
        xs = []
        for p in range(n):
            g = torch.Generator().manual_seed(11 * p + m_shard)
            xs.append((torch.randn(m_shard, K, generator=g) * 0.5).to(torch.bfloat16))
        g = torch.Generator().manual_seed(500 + me)
        w = (torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16).to(dev)
        for rep in range(3):  # repeated calls exercise the epoch counters
            tp.ag_input(K).copy_(xs[me].to(dev))
            torch.cuda.synchronize()
            shm.barrier_all()
            before = gemm.gemm_error_count()
            out = tp.ag_gemm(w)
            _ok()
            assert gemm.gemm_error_count() == before
            want = torch.cat(xs).float().to(dev) @ w.float().t()
            err = (out.float() - want).abs().max().item()
            assert err <= 1e-2 * want.abs().max().item() + 0.05, ("ag_gemm", m_shard, K, N, rep, err)
        # GEMM -> reduce-scatter: a is [n * m_shard, K_local] per rank with its own K slice
        ws, as_ = [], []
        for p in range(n):
            g = torch.Generator().manual_seed(900 + p)
            as_.append((torch.randn(n * m_shard, K, generator=g) * 0.5).to(torch.bfloat16))
            ws.append((torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16))
        a_dev, w_dev = as_[me].to(dev), ws[me].to(dev)
        for rep in range(3):
            before = gemm.gemm_error_count()
            out = tp.gemm_rs(a_dev, w_dev)
            _ok()
            assert gemm.gemm_error_count() == before
            total = sum(a.float() @ wv.float().t() for a, wv in zip(as_, ws))
            want = total[me * m_shard:(me + 1) * m_shard].to(dev)
            err = (out.float() - want).abs().max().item()
            # every rank's partial is rounded to bf16 before the sum
            assert err <= 2e-2 * want.abs().max().item() + 0.1, ("gemm_rs", m_shard, K, N, rep, err)
        shm.barrier_all()
    shm.finalize()


def gpu_models():
    """Tensor-parallel MLP and expert-parallel MoE feed-forward layer against plain fp32 PyTorch
    evaluations of the same layers (weights are rebuilt from seeds on every rank)."""
    from rocshmem_b200.models import moe_ffn, tp_mlp
    from rocshmem_b200.ops import gemm, moe
    _init("2G")
    me, n = RANK, WORLD
    dev = shm.device()
    # -- TP MLP
    d_model, d_ff, m_shard = 1024, 512 * n, 256
    mlp = tp_mlp.TensorParallelMLP(d_model, d_ff, m_shard, seed=3)
    xs = [(torch.randn(m_shard, d_model, generator=torch.Generator().manual_seed(40 + p)) * 0.5).to(torch.bfloat16)
          for p in range(n)]
    want = tp_mlp.reference_forward(torch.cat(xs), n, d_model, d_ff, seed=3)[me * m_shard:(me + 1) * m_shard]
    for rep in range(2):
        before = gemm.gemm_error_count()
        out = mlp(xs[me].to(dev))
        _ok()
        assert gemm.gemm_error_count() == before
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 0.05, ("tp_mlp", rep, err)
        shm.barrier_all()
    # -- TP MLP with block-scaled e4m3 GEMMs (e4m3 rows and their scales cross NVLink)
    d_ff8 = 512 * n
    mlp8 = tp_mlp.TensorParallelMLPFp8(d_model, d_ff8, m_shard, seed=8)
    want8 = tp_mlp.reference_forward_fp8(torch.cat(xs), n, d_model, d_ff8, seed=8)[me * m_shard:(me + 1) * m_shard]
    for rep in range(2):
        before = gemm.gemm_error_count()
        out = mlp8(xs[me].to(dev))
        _ok()
        assert gemm.gemm_error_count() == before
        err = (out.float().cpu() - want8).abs().max().item()
        assert err <= 5e-2 * want8.abs().max().item() + 0.05, ("tp_mlp_fp8", rep, err)
        shm.barrier_all()
    # -- MoE feed-forward: bf16 experts, block-scaled e4m3 experts (the default here), and the low-latency kernels
    E, K, H, I, T = 8 * n, 4, 1024, 512, 160 + 8 * me
    for kw, tol in ((dict(fp8_experts=False), (3e-2, 0.02)), (dict(), (5e-2, 0.03)),
                    (dict(low_latency=True, layout="slotted"), (5e-2, 0.03))):
        layer = moe_ffn.MoEFeedForward(E, K, H, I, max_tokens=256, seed=5, **kw)
        for rep in range(2):
            g = torch.Generator().manual_seed(77 * rep + me)
            x = torch.randn(T, H, generator=g).to(torch.bfloat16)
            idx, w = moe.make_routing(T, E, K, 1000 * rep + me)
            if rep == 1:
                idx[::9, -1] = -1
            before = gemm.gemm_error_count()
            out = layer(x.to(dev), idx.to(dev), w.to(dev))
            _ok()
            assert gemm.gemm_error_count() == before
            want = moe_ffn.reference_forward(x, idx, w, H, I, seed=5, fp8_experts=layer.fp8_experts)
            err = (out.float().cpu() - want).abs().max().item()
            assert err <= tol[0] * want.abs().max().item() + tol[1], ("moe_ffn", kw, rep, err, want.abs().max().item())
            shm.barrier_all()
        layer.destroy()
    shm.finalize()


SCENARIOS = {f.__name__: f for f in (gpu_device_suite, gpu_library_collectives, gpu_team_nvls, gpu_proxied_collectives, gpu_moe,
                                     gpu_tp_fused, gpu_models)}
