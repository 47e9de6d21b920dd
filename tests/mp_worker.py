"""One PE process of a multi-process test scenario (started by mp_util.run_ranks).

Environment: RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT as torchrun sets them, ROCSHMEM_TEST_TMP a
scratch directory shared by the ranks, ROCSHMEM_TEST_BACKEND 'host' (default) or 'cuda'.
"""
import os
import sys
import time

import torch

import rocshmem_b200 as shm
from rocshmem_b200.ops import collectives as coll

RANK = int(os.environ["RANK"])
WORLD = int(os.environ["WORLD_SIZE"])
TMP = os.environ.get("ROCSHMEM_TEST_TMP", "/tmp")
BACKEND = os.environ.get("ROCSHMEM_TEST_BACKEND", "host")


def init(heap="64M", **kw):
    shm.init(heap_size=heap, backend=BACKEND, timeout_s=float(os.environ.get("ROCSHMEM_TEST_TIMEOUT", "60")), **kw)
    assert shm.n_pes() == WORLD and shm.my_pe() == RANK


def dev():
    return shm.device()


def host_plumbing():
    """64 MiB heap, 1 MiB int64 buffers filled with pe * 2^32 + i: put to the right neighbour, get it
    back, fetch-add on a symmetric counter, barrier; everything bit-exact."""
    init("64M")
    n = (1 << 20) // 8
    me, npes = shm.my_pe(), shm.n_pes()
    src = shm.empty(n, torch.int64)
    dst = shm.zeros(n, torch.int64)
    back = torch.zeros(n, dtype=torch.int64, device=dev())
    counter = shm.zeros(1, torch.int64)
    src.copy_(torch.arange(n, dtype=torch.int64, device=dev()) + (me << 32))
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    right, left = (me + 1) % npes, (me - 1) % npes
    shm.putmem(dst, src, right)
    shm.barrier_all()
    expect = torch.arange(n, dtype=torch.int64) + (left << 32)
    assert torch.equal(dst.cpu(), expect), "put pattern mismatch"
    shm.getmem(back, dst, right)
    assert torch.equal(back.cpu(), torch.arange(n, dtype=torch.int64) + (me << 32)), "get pattern mismatch"
    olds = [shm.atomic_fetch_add(counter, 1, 0) for _ in range(10)]
    assert all(0 <= o < 10 * npes for o in olds) and len(set(olds)) == 10
    shm.barrier_all()
    if me == 0:
        assert int(counter.cpu()[0]) == 10 * npes
    # compare-and-swap election: exactly one PE wins
    flag = shm.zeros(1, torch.int64)
    won = shm.atomic_compare_swap(flag, 0, me + 1, 0) == 0
    shm.barrier_all()
    winner = shm.atomic_fetch(flag, 0)
    assert (winner == me + 1) == won
    shm.free(flag)
    shm.finalize()


def store_bootstrap():
    """Same runtime, bootstrapped through a torch.distributed TCPStore."""
    import datetime
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), WORLD, RANK == 0,
                          timeout=datetime.timedelta(seconds=60))
    shm.init(store=store, heap_size="8M", backend=BACKEND)
    x = shm.zeros(16, torch.float32)
    x.fill_(float(RANK + 1))
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    got = torch.zeros(16, dtype=torch.float32, device=dev())
    shm.getmem(got, x, (RANK + 1) % WORLD)
    assert float(got.cpu()[0]) == float((RANK + 1) % WORLD + 1)
    shm.barrier_all()
    shm.finalize()


def teams():
    init("16M")
    me, npes = shm.my_pe(), shm.n_pes()
    world = shm.team_world()
    assert world.n_pes() == npes and world.my_pe() == me
    even = world.split_strided(0, 2, (npes + 1) // 2)
    if me % 2 == 0:
        assert even.valid and even.my_pe() == me // 2 and even.n_pes() == (npes + 1) // 2
        assert even.translate_pe(even.my_pe(), world) == me
        a = None
    else:
        assert not even.valid
    src = shm.zeros(64, torch.int64)
    dst = shm.zeros(64, torch.int64)
    src.fill_(me + 1)
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    if even.valid:
        assert coll.reduce(dst, src, shm.OP_SUM, even) == 0
        expect = sum(p + 1 for p in range(0, npes, 2))
        assert int(dst.cpu()[0]) == expect and int(dst.cpu()[-1]) == expect
    shm.barrier_all()
    # invalid requests
    for bad in ((0, 1, npes + 1), (npes, 1, 1), (0, 0, 1), (-1, 1, 1)):
        try:
            world.split_strided(*bad)
            raise AssertionError(f"split {bad} should have been rejected")
        except ValueError:
            pass
    # sub-split of the even team: its first member alone
    if even.valid:
        solo = even.split_strided(0, 1, 1)
        assert solo.valid == (even.my_pe() == 0)
        if solo.valid:
            assert solo.n_pes() == 1 and solo.translate_pe(0, world) == 0
            solo.destroy()
        even.destroy()
    # 39 duplicates of the world fit (slot 0 is TEAM_WORLD), the 40th is refused
    dups = [world.split_strided(0, 1, npes) for _ in range(39)]
    assert all(d.valid for d in dups)
    try:
        world.split_strided(0, 1, npes)
        raise AssertionError("40th team should fail")
    except RuntimeError:
        pass
    # every duplicate is usable and independent
    assert coll.reduce(dst, src, shm.OP_MAX, dups[17]) == 0
    assert int(dst.cpu()[3]) == npes
    for d in dups:
        d.destroy()
    again = world.split_strided(0, 1, npes)
    assert again.valid
    again.destroy()
    shm.barrier_all()
    shm.finalize()


def team_multicast_standin():
    """Set-up and tear-down of the world's and of split teams' multicast objects, with the host provider's stand-in for
    the NVLink object: every member ends with a mapping, or (when one member's step fails) nobody does; destroying
    such a team is collective; a slot is reused; teams are still alive at finalize. The failing step comes from the
    environment of one rank (ROCSHMEM_HOST_FAKE_MULTICAST_FAIL, set by the test)."""
    if os.environ.get("FAKE_MC_FAIL_RANK") == str(RANK):
        os.environ["ROCSHMEM_HOST_FAKE_MULTICAST_FAIL"] = os.environ["FAKE_MC_FAIL_SPEC"]
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    world = shm.team_world()
    spec = os.environ.get("EXPECT_MULTICAST", "")      # "world,lower,upper,even" : which objects must exist
    expect = set(spec.split(",")) if spec else set()
    assert shm.nvls_available() == ("world" in expect), (shm.nvls_available(), expect)
    assert world.has_nvls() == ("world" in expect)
    half = n // 2
    src, dst = shm.zeros(64, torch.int64), shm.zeros(64, torch.int64)
    src.fill_(me + 1)
    shm.barrier_all()
    lower = world.split_strided(0, 1, half)
    upper = world.split_strided(half, 1, n - half)
    even = world.split_strided(0, 2, (n + 1) // 2)
    for name, t, members in (("lower", lower, list(range(half))), ("upper", upper, list(range(half, n))),
                             ("even", even, list(range(0, n, 2)))):
        assert t.valid == (me in members), name
        if not t.valid:
            continue
        want = name in expect and len(members) >= 2
        assert t.has_nvls() == want, (name, t.has_nvls(), want)
        # the team works either way
        assert coll.reduce(dst, src, shm.OP_SUM, t) == 0
        assert int(dst.cpu()[0]) == sum(p + 1 for p in members), name
    shm.barrier_all()
    # destroy (collective for teams with an object) and split again into the freed slots, with other members
    for t in (lower, upper, even):
        if t.valid:
            t.destroy()
    shm.barrier_all()
    if n >= 3:
        rest = world.split_strided(1, 1, n - 1)
        if me >= 1:
            assert rest.valid and rest.has_nvls() == ("rest" in expect), (rest.has_nvls(), expect)
            assert coll.reduce(dst, src, shm.OP_MAX, rest) == 0 and int(dst.cpu()[5]) == n
        else:
            assert not rest.valid
    dup = world.split_strided(0, 1, n)          # same members as the world: shares the world's mapping
    assert dup.valid and dup.has_nvls() == ("world" in expect)
    shm.barrier_all()
    shm.finalize()     # "rest" and "dup" are still alive


def collectives_host():
    init("64M")
    me, npes = shm.my_pe(), shm.n_pes()
    world = shm.team_world()
    for dtype, n in ((torch.float32, 1000), (torch.int32, 17), (torch.float64, 4096), (torch.int64, 1),
                     (torch.bfloat16, 513), (torch.int16, 129)):
        src = shm.zeros(n, dtype)
        dst = shm.zeros(n, dtype)
        gen = torch.Generator().manual_seed(1234 + me)
        if dtype.is_floating_point:
            host = torch.randn(n, generator=gen, dtype=torch.float64).to(dtype)
        else:
            host = torch.randint(-50, 50, (n,), generator=gen, dtype=torch.int64).to(dtype)
        src.copy_(host.to(dev()))
        if shm.is_cuda():
            torch.cuda.synchronize()
        shm.barrier_all()
        alls = []
        for p in range(npes):
            g = torch.Generator().manual_seed(1234 + p)
            if dtype.is_floating_point:
                alls.append(torch.randn(n, generator=g, dtype=torch.float64).to(dtype))
            else:
                alls.append(torch.randint(-50, 50, (n,), generator=g, dtype=torch.int64).to(dtype))
        ops = [(shm.OP_SUM, lambda xs: torch.stack(xs).sum(0)), (shm.OP_MAX, lambda xs: torch.stack(xs).max(0).values),
               (shm.OP_MIN, lambda xs: torch.stack(xs).min(0).values)]
        if not dtype.is_floating_point:
            def fold(fn):
                def f(xs):
                    acc = xs[0].clone()
                    for x in xs[1:]:
                        acc = fn(acc, x)
                    return acc
                return f
            ops += [(shm.OP_AND, fold(torch.bitwise_and)), (shm.OP_OR, fold(torch.bitwise_or)),
                    (shm.OP_XOR, fold(torch.bitwise_xor))]
        for op, ref_fn in ops:
            assert coll.reduce(dst, src, op, world) == 0
            ref = ref_fn([a.to(torch.float64) if dtype.is_floating_point else a.to(torch.int64) for a in alls])
            got = dst.cpu().to(ref.dtype)
            if dtype.is_floating_point:
                tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
                assert torch.allclose(got, ref, rtol=tol, atol=tol * npes), (dtype, op)
            else:
                assert torch.equal(got, ref.to(torch.int64)), (dtype, op)
        # in place
        assert coll.reduce(src, src, shm.OP_SUM, world) == 0
        shm.free(dst)
        shm.free(src)
    # broadcast: the root's dest stays untouched
    src = shm.zeros(300, torch.int32)
    dst = shm.zeros(300, torch.int32)
    src.fill_(1000 + me)
    dst.fill_(-1)
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    root = npes - 1
    assert coll.broadcast(dst, src, root) == 0
    want = -1 if me == root else 1000 + root
    assert torch.all(dst.cpu() == want)
    # fcollect and alltoall
    gat = shm.zeros(300 * npes, torch.int32)
    assert coll.fcollect(gat, src) == 0
    g = gat.cpu().view(npes, 300)
    assert all(torch.all(g[p] == 1000 + p) for p in range(npes))
    a2a_src = shm.zeros(npes * 7, torch.int32)
    a2a_dst = shm.zeros(npes * 7, torch.int32)
    a2a_src.copy_((torch.arange(npes * 7, dtype=torch.int32) + 100 * me).to(dev()))
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    assert coll.alltoall(a2a_dst, a2a_src) == 0
    got = a2a_dst.cpu().view(npes, 7)
    for p in range(npes):
        assert torch.equal(got[p], torch.arange(7, dtype=torch.int32) + me * 7 + 100 * p)
    # active-set reduction over PEs {0, 2, ...}: only the members call
    if me % 2 == 0 and npes >= 2:
        s2 = src  # 1000 + me
        rc = shm.runtime._C().reduce_active_set(dst.data_ptr(), s2.data_ptr(), 300, shm.runtime.dtype_code(torch.int32),
                                                shm.OP_SUM, 0, 1, (npes + 1) // 2)
        assert rc == 0
        assert int(dst.cpu()[0]) == sum(1000 + p for p in range(0, npes, 2))
    shm.barrier_all()
    shm.finalize()


def wait_and_signal():
    """Host wait_until / test family between processes."""
    init("8M")
    me, npes = shm.my_pe(), shm.n_pes()
    flags = shm.zeros(npes, torch.int64)
    one = torch.ones(1, dtype=torch.int64, device=dev()) * (me + 1)
    for p in range(npes):
        shm.putmem(flags[me:me + 1], one, p)
    shm.wait_until_all(flags, shm.CMP_GT, 0)
    assert shm.test(flags, shm.CMP_EQ, 1, index=0)
    assert shm.wait_until_any(flags, shm.CMP_EQ, npes) == npes - 1
    assert sorted(shm.wait_until_some(flags, shm.CMP_GE, 1)) == list(range(npes))
    shm.wait_until_all(flags, shm.CMP_EQ, [p + 1 for p in range(npes)])
    assert shm.wait_until_any(flags, shm.CMP_EQ, 1, status=[1] * npes) == -1
    shm.barrier_all()
    # a wait that nobody satisfies gives up after the configured budget
    shm.set_wait_timeout_ms(200)
    t0 = time.time()
    assert shm.wait_until(flags, shm.CMP_EQ, 424242) == shm.ERROR
    assert 0.15 < time.time() - t0 < 5.0
    err = shm.get_error()
    assert err["kind"] == 1 and err["expected"] == 424242
    shm.clear_error()
    assert shm.get_error()["count"] == 0
    shm.barrier_all()
    shm.finalize()


def late_rank():
    """Rank 1 never joins: the others' init must raise within the bootstrap time-out, not hang."""
    if RANK == 1:
        time.sleep(float(sys.argv[2]) if len(sys.argv) > 2 else 4.0)
        return
    os.environ["ROCSHMEM_TEST_TIMEOUT"] = "2"
    t0 = time.time()
    try:
        init("8M")
    except Exception as e:  # BootstrapError surfaces as RuntimeError
        assert "timed out" in str(e) or "Timeout" in str(e) or "wait" in str(e).lower(), str(e)
        assert time.time() - t0 < 30
        print("detected:", str(e)[:120])
        return
    raise AssertionError("init succeeded although a rank never joined")


def rank_leaves():
    """A rank leaves between steps; the others learn of it from the membership record in the store
    before their next collective and shrink to a team without it."""
    from rocshmem_b200.parallel.membership import Membership
    init("8M")
    me, npes = shm.my_pe(), shm.n_pes()
    mem = Membership.from_env(prefix="t1")
    x = shm.zeros(8, torch.int64)
    y = shm.zeros(8, torch.int64)
    x.fill_(me + 1)
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    assert coll.reduce(y, x) == 0
    leaver = npes - 1
    if me == leaver:
        # Leaves with nothing in flight: after the step, before the next one starts.
        mem.announce_leave()
        shm.runtime._C().quiet()
        # The process stays until the others have stopped using its memory.
        mem.wait_for("survivors-done", timeout_s=60)
        return
    alive = mem.wait_for_change(expected_alive=npes - 1, timeout_s=30)
    assert alive == list(range(npes - 1)), alive
    # Survivors reduce over an active set that excludes the leaver: only its members take part in setting it up,
    # so the absent rank is not needed.
    rc = shm.runtime._C().reduce_active_set(y.data_ptr(), x.data_ptr(), 8, shm.runtime.dtype_code(torch.int64),
                                            shm.OP_SUM, 0, 0, npes - 1)
    assert rc == 0 and int(y.cpu()[0]) == sum(range(1, npes))
    if me == 0:
        mem.post("survivors-done")


def team_member_leaves():
    """A team with a multicast object of its own (the host provider's stand-in) loses a member between steps: the
    survivor's collective team_destroy gives up after the rendezvous time-out, releases the object and returns; the
    process then finishes without the absent rank."""
    import time
    init("8M")
    me, n = shm.my_pe(), shm.n_pes()
    pair = shm.team_world().split_strided(0, 1, 2)
    if me < 2:
        assert pair.valid and pair.has_nvls()
    shm.barrier_all()
    if me == 1:
        return                      # leaves between steps, nothing in flight, without destroying its team
    if me == 0:
        t0 = time.time()
        pair.destroy()              # meets nobody: bounded by the rendezvous time-out, then the mapping goes
        waited = time.time() - t0
        assert 1.0 < waited < 40.0, waited
        assert not pair.valid
    # PE 2 was never a member and is not involved


def proxy_collectives():
    """The reverse-offload command ring executing the host forms of fence, P, broadcast, reduce, fcollect and
    alltoall (each rank submits the command to its own proxy thread, like a device kernel would)."""
    from rocshmem_b200 import runtime as rt
    init("16M")
    C = rt._C()
    me, npes = shm.my_pe(), shm.n_pes()
    FENCE, BROADCAST, REDUCE, FCOLLECT, ALLTOALL, P = 8, 9, 10, 11, 12, 13
    I64 = 6  # ROCSHMEM_I64
    p = C.proxy_start()
    try:
        n = 64
        src = shm.zeros(n * npes, torch.int64)
        dst = shm.zeros(n * npes, torch.int64)
        src.copy_((torch.arange(n * npes) + 1000 * me).to(dev()))
        shm.barrier_all()
        sub = lambda *a: C.proxy_submit(p, *a, True, 20000)
        assert sub(FENCE, 0, 0, 0, 0, 0, 0, 0)[0] == 0
        # reduce: sum over ranks of (i + 1000 r)
        rc, status = sub(REDUCE, 0, dst.data_ptr(), src.data_ptr(), n, I64, shm.OP_SUM, 8)
        assert rc == 0 and status == 0
        want = torch.arange(n) * npes + 1000 * sum(range(npes))
        assert torch.equal(dst.cpu()[:n], want)
        shm.barrier_all()
        # broadcast from the last rank: everybody else receives its src
        dst.zero_()
        shm.barrier_all()
        root = npes - 1
        assert sub(BROADCAST, root, dst.data_ptr(), src.data_ptr(), n * 8, 0, 0, 1)[0] == 0
        got = dst.cpu()[:n]
        assert torch.equal(got, torch.zeros(n, dtype=torch.int64) if me == root else torch.arange(n) + 1000 * root)
        shm.barrier_all()
        # fcollect: block r of dst is rank r's first n elements
        assert sub(FCOLLECT, 0, dst.data_ptr(), src.data_ptr(), n * 8, 0, 0, 1)[0] == 0
        got = dst.cpu().view(npes, n)
        assert all(torch.equal(got[r], torch.arange(n) + 1000 * r) for r in range(npes))
        shm.barrier_all()
        # alltoall: block r of dst is rank r's block `me`
        assert sub(ALLTOALL, 0, dst.data_ptr(), src.data_ptr(), n * 8, 0, 0, 1)[0] == 0
        got = dst.cpu().view(npes, n)
        assert all(torch.equal(got[r], torch.arange(n) + me * n + 1000 * r) for r in range(npes))
        shm.barrier_all()
        # P: one element by value to the right-hand neighbour
        cell = shm.zeros(1, torch.int64)
        shm.barrier_all()
        assert sub(P, (me + 1) % npes, cell.data_ptr(), 0, 4242 + me, 0, 0, 8)[0] == 0
        shm.barrier_all()
        assert int(cell.cpu()[0]) == 4242 + (me - 1) % npes
        # collectives of a sub-team: the command names the team by its sync-pool slot
        BARRIER = 6
        half = max(1, npes // 2)
        lower = shm.team_world().split_strided(0, 1, half)
        upper = shm.team_world().split_strided(half, 1, npes - half) if npes > half else None
        mine = lower if lower.valid else upper
        slot = C.team_slot(mine.handle)
        assert slot >= 1
        members = list(range(half)) if lower.valid else list(range(half, npes))
        subt = lambda *a: C.proxy_submit(p, *a, True, 20000, slot)
        rc, status = subt(REDUCE, 0, dst.data_ptr(), src.data_ptr(), n, I64, shm.OP_SUM, 8)
        assert rc == 0 and status == 0
        assert torch.equal(dst.cpu()[:n], torch.arange(n) * len(members) + 1000 * sum(members))
        rc, status = subt(BARRIER, 0, 0, 0, 0, 0, 0, 0)
        assert rc == 0 and status == 0
        # a slot that no team owns fails the command instead of running it on the wrong team
        rc, status = C.proxy_submit(p, REDUCE, 0, dst.data_ptr(), src.data_ptr(), n, I64, shm.OP_SUM, 8, True, 20000, 37)
        assert rc == 0 and status == 1
        shm.barrier_all()
        for t in (lower, upper):
            if t is not None and t.valid:
                t.destroy()
    finally:
        C.proxy_stop(p)
    shm.barrier_all()
    shm.finalize()


def ep_host():
    """Expert-parallel dispatch / combine through the host API: layout and records against the reference routing,
    then a round trip (identity experts) against the de-quantised input."""
    from rocshmem_b200.ops import moe, moe_host
    init("64M")
    me, P = shm.my_pe(), shm.n_pes()
    E, K, H, T = 4 * P, 3, 256, 37 + me
    used_before = shm.heap_info()["used"]
    d = moe_host.HostEpDispatcher(E, K, H, max_tokens=64)
    for rep in range(2):
        routing = [moe.make_routing(37 + r, E, K, seed=10 * rep + r) for r in range(P)]
        if rep == 1:
            for idx, _ in routing:
                idx[::4, -1] = -1
        xs = [torch.randn(37 + r, H, generator=torch.Generator().manual_seed(100 * rep + r)).to(torch.bfloat16)
              for r in range(P)]
        idx, w = routing[me]
        res = d.dispatch(xs[me].to(dev()), idx, w)
        want_rows = moe.ref_dispatch([r[0] for r in routing], P, E)[me]
        info = res.recv_info.cpu().tolist()
        assert info[0] == len(want_rows)
        pos = 0
        for s in range(P):
            mine = [t for ss, t in want_rows if ss == s]
            assert info[1 + s] == pos and info[1 + P + s] == len(mine)
            rows = slice(pos, pos + len(mine))
            pos += len(mine)
            if not mine:
                continue
            assert res.src_token()[rows].cpu().tolist() == mine and set(res.src_rank()[rows].cpu().tolist()) == {s}
            q, sc = moe.ref_quantize_1x128(xs[s][mine])
            assert torch.equal(res.recv_x[rows].cpu().view(torch.uint8), q.view(torch.uint8))
            assert torch.allclose(res.recv_scales[rows].cpu(), sc)
            src_idx, src_w = routing[s]
            epr = E // P
            want_local = torch.where(src_idx[mine] // epr == me, src_idx[mine] % epr, torch.full_like(src_idx[mine], -1))
            want_local = torch.where(src_idx[mine] >= 0, want_local, torch.full_like(want_local, -1))
            assert torch.equal(res.local_expert_idx()[rows].cpu(), want_local.to(torch.int32))
            assert torch.equal(res.gate_weights()[rows].cpu(), src_w[mine])
        per_expert = res.rows_per_expert().cpu().tolist()
        assert sum(per_expert) == int((res.local_expert_idx()[:info[0]].cpu() >= 0).sum())
        # identity experts: every rank returns the de-quantised rows it received
        y = d.result_buffer()
        n_rows = info[0]
        y[:n_rows].copy_(moe.ref_dequantize_1x128(res.recv_x[:n_rows].cpu(), res.recv_scales[:n_rows].cpu()).to(torch.bfloat16).to(dev()))
        out = d.combine(y, idx, w, xs[me].shape[0])
        q, sc = moe.ref_quantize_1x128(xs[me])
        xd = moe.ref_dequantize_1x128(q, sc).to(torch.bfloat16).float()
        gate = torch.where(idx >= 0, w, torch.zeros_like(w)).sum(dim=1, keepdim=True)
        assert torch.allclose(out.float(), xd * gate, rtol=2e-2, atol=2e-2), rep
    shm.barrier_all()
    assert shm.heap_info()["used"] > used_before
    d.destroy()                                  # every symmetric buffer goes back to the heap
    assert shm.heap_info()["used"] == used_before
    shm.finalize()


def moe_layer_host():
    """The MoE feed-forward layer over the host-API dispatcher against the single-process fp32 evaluation."""
    from rocshmem_b200.models import moe_ffn
    from rocshmem_b200.ops import moe
    init("64M")
    me, P = shm.my_pe(), shm.n_pes()
    E, K, H, I, T = 2 * P, 2, 256, 128, 29 + 2 * me
    used_before = shm.heap_info()["used"]
    layer = moe_ffn.HostMoEFeedForward(E, K, H, I, max_tokens=64, seed=9)
    for rep in range(2):
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(50 * rep + me)).to(torch.bfloat16)
        idx, w = moe.make_routing(T, E, K, seed=7 * rep + me)
        if rep:
            idx[::5, -1] = -1
        out = layer(x.to(dev()), idx, w)
        want = moe_ffn.reference_forward(x, idx, w, H, I, seed=9)
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 0.02, (rep, err)
    shm.barrier_all()
    layer.destroy()
    assert shm.heap_info()["used"] == used_before
    shm.finalize()


def parallel_layout():
    """A 2 x 2 process grid: row teams (tensor / expert parallel), column teams (data parallel), a reduction over
    each, and a pipeline channel between the first and the last PE."""
    from rocshmem_b200.parallel import layout as pl, pipeline
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    assert n == 4
    lay = pl.ParallelLayout(inner=2)
    assert (lay.row, lay.col, lay.dp, lay.inner) == (me // 2, me % 2, 2, 2)
    assert lay.inner_team.n_pes() == 2 and lay.inner_team.my_pe() == me % 2
    assert lay.dp_team.n_pes() == 2 and lay.dp_team.my_pe() == me // 2
    assert lay.inner_team.translate_pe(1, shm.team_world()) == (me // 2) * 2 + 1
    assert lay.dp_team.translate_pe(1, shm.team_world()) == 2 + me % 2
    src = shm.zeros(8, torch.int64)
    dst = shm.zeros(8, torch.int64)
    src.fill_(1 << me)
    shm.barrier_all()
    assert coll.reduce(dst, src, shm.OP_SUM, lay.inner_team) == 0
    row = me // 2
    assert int(dst.cpu()[0]) == (1 << (2 * row)) + (1 << (2 * row + 1))
    assert coll.reduce(dst, src, shm.OP_SUM, lay.dp_team) == 0
    assert int(dst.cpu()[0]) == (1 << (me % 2)) + (1 << (2 + me % 2))
    shm.barrier_all()
    # pipeline: PE 0 -> PE 3, three messages in order, back-pressure through the acknowledgement counter
    used_before = shm.heap_info()["used"]
    ch = pipeline.P2PChannel((16,), torch.float32, src_pe=0, dst_pe=3)
    shm.barrier_all()
    for i in range(3):
        if me == 0:
            ch.send(torch.full((16,), float(i + 1)).to(dev()))
        elif me == 3:
            got = ch.recv()
            assert torch.all(got.cpu() == float(i + 1)), (i, got)
    shm.barrier_all()
    ch.destroy()
    assert shm.heap_info()["used"] == used_before
    lay.destroy()
    shm.finalize()


def stress_host():
    """Back-to-back collectives without barriers in between, repeated team creation and destruction, and many
    context create / destroy cycles (the reference's SOS tests shmem_team_b2b_collectives, shmem_team_reuse_teams,
    many-ctx)."""
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    world = shm.team_world()
    src = shm.zeros(64 * n, torch.int64)
    dst = shm.zeros(64 * n, torch.int64)
    for it in range(30):
        src.copy_((torch.arange(64 * n) + it + 100 * me).to(dev()))
        if shm.is_cuda():
            torch.cuda.synchronize()
        assert coll.reduce(dst[:64], src[:64], shm.OP_SUM, world) == 0
        assert torch.equal(dst.cpu()[:64], (torch.arange(64) + it) * n + 100 * sum(range(n)))
        assert coll.fcollect(dst, src[:64], world) == 0
        got = dst.cpu().view(n, 64)
        assert all(int(got[r][5]) == 5 + it + 100 * r for r in range(n))
        assert coll.broadcast(dst[:64], src[:64], it % n, world) == 0
        if me != it % n:
            assert int(dst.cpu()[7]) == 7 + it + 100 * (it % n)
    before = shm.runtime._C().num_user_teams()
    for it in range(25):
        half = world.split_strided(0, 1, max(1, n // 2))
        rest = world.split_strided(max(1, n // 2), 1, n - max(1, n // 2)) if n > 1 else None
        mine = half if half.valid else rest
        if mine is not None and mine.valid:
            assert coll.reduce(dst[:8], src[:8], shm.OP_MAX, mine) == 0
        for t in (half, rest):
            if t is not None and t.valid:
                t.destroy()
    assert shm.runtime._C().num_user_teams() == before
    shm.barrier_all()   # the team reductions above write dst too
    for it in range(100):
        c = shm.Context()
        shm.putmem(dst[:8], torch.full((8,), it, dtype=torch.int64).to(dev()), (me + 1) % n, ctx=c)
        c.quiet()
        c.destroy()
    shm.barrier_all()
    assert int(dst.cpu()[0]) == 99
    shm.barrier_all()
    shm.finalize()


def host_algorithms():
    """Bruck and clustered schedules of alltoall / fcollect against the expected layout, for block sizes below and
    at the plan's capacity."""
    from rocshmem_b200.ops.host_algorithms import HostCollectivePlan, choose_algorithm, cluster_size
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    plan = HostCollectivePlan(max_block_bytes=96)
    assert plan.cluster == cluster_size(n) and n % plan.cluster == 0
    for elems in (1, 5, 12):                     # int64 blocks of 8, 40 and 96 bytes
        src = shm.zeros(n * elems, torch.int64)
        dst = shm.zeros(n * elems, torch.int64)
        one = shm.zeros(elems, torch.int64)
        src.copy_((1000 * me + torch.arange(n * elems)).to(dev()))
        one.copy_((7000 * me + torch.arange(elems)).to(dev()))
        want_a2a = torch.cat([1000 * p + me * elems + torch.arange(elems) for p in range(n)])
        want_fc = torch.cat([7000 * p + torch.arange(elems) for p in range(n)])
        for algo in ("linear", "bruck", "clustered", "auto"):
            dst.zero_()
            used = plan.alltoall(dst, src, algo)
            assert torch.equal(dst.cpu(), want_a2a), (algo, used, elems, dst.cpu(), want_a2a)
            dst.zero_()
            used = plan.fcollect(dst, one, algo)
            assert torch.equal(dst.cpu(), want_fc), (algo, used, elems, dst.cpu(), want_fc)
    plan.destroy()
    assert choose_algorithm(2, 8) == "linear" and choose_algorithm(8, 1 << 20) == "linear"
    assert choose_algorithm(64, 8) in ("bruck", "clustered")
    shm.barrier_all()
    shm.finalize()


def threads_host():
    """Several host threads per process, each with its own context: an all-to-all of puts from every thread
    (the reference's SOS test mt_a2a), a chain of waits where a thread of PE p waits for the matching thread of
    PE p - 1 (thread_wait), and one large put / get pair (bigput / bigget)."""
    import threading
    init("160M")
    me, n = shm.my_pe(), shm.n_pes()
    T, W = 4, 32
    dst = shm.zeros(n * T * W, torch.int64)      # [source pe][thread][W]
    flags = shm.zeros(T, torch.int64)
    errors = []
    shm.barrier_all()

    def work(t):
        try:
            ctx = shm.Context()
            for j in range(n):
                pe = (me + j) % n
                val = torch.full((W,), 100 * me + t, dtype=torch.int64).to(dev())
                shm.putmem(dst[(me * T + t) * W:(me * T + t + 1) * W], val, pe, ctx=ctx)
            ctx.quiet()
            # chain: PE 0 starts, everyone else waits for its predecessor's thread t, then passes on
            if me > 0:
                assert shm.wait_until(flags, shm.CMP_EQ, 1 + t, index=t) == 0
            if me + 1 < n:
                shm.atomic_swap(flags, 1 + t, me + 1, index=t, ctx=ctx)
            ctx.destroy()
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append((t, repr(e)))

    threads = [threading.Thread(target=work, args=(t,)) for t in range(T)]
    [t.start() for t in threads]
    [t.join(120) for t in threads]
    assert not errors, errors
    shm.barrier_all()
    got = dst.cpu().view(n, T, W)
    for p in range(n):
        for t in range(T):
            assert torch.all(got[p, t] == 100 * p + t), (p, t, got[p, t][:4])
    # one large transfer each way (32 MiB)
    big = shm.zeros(4 << 20, torch.int64)
    back = shm.zeros(4 << 20, torch.int64)
    pattern = (torch.arange(4 << 20, dtype=torch.int64) * 3 + me).to(dev())
    shm.putmem(big, pattern, (me + 1) % n)
    shm.barrier_all()
    left = (me - 1) % n
    assert torch.equal(big.cpu(), torch.arange(4 << 20, dtype=torch.int64) * 3 + left)
    shm.getmem(back, big, (me + 1) % n)
    assert torch.equal(back.cpu(), torch.arange(4 << 20, dtype=torch.int64) * 3 + me)
    shm.barrier_all()
    shm.finalize()


def collective_baselines():
    """The torch.distributed wrappers that the benchmarks time against (rocshmem_b200.baselines), over gloo: the same
    calling conventions as ops.collectives, results against what every rank can compute itself."""
    import torch.distributed as dist
    from rocshmem_b200 import baselines
    dist.init_process_group("gloo", rank=RANK, world_size=WORLD)
    me, n = RANK, WORLD
    src = torch.arange(8, dtype=torch.float32) + 10 * me
    dst = torch.zeros(8)
    baselines.allreduce(dst, src)
    assert torch.equal(dst, torch.arange(8, dtype=torch.float32) * n + 10 * sum(range(n)))
    assert torch.equal(src, torch.arange(8, dtype=torch.float32) + 10 * me)        # the source is left alone
    baselines.allreduce(src, src)                                                  # in place
    assert torch.equal(src, dst)
    gathered = torch.zeros(4 * n)
    baselines.allgather(gathered, torch.full((4,), float(me)))
    assert torch.equal(gathered.view(n, 4), torch.arange(n, dtype=torch.float32).view(n, 1).expand(n, 4))
    a2a = torch.zeros(2 * n)
    baselines.alltoall(a2a, torch.arange(2 * n, dtype=torch.float32) + 100 * me)
    want = torch.cat([torch.arange(2 * me, 2 * me + 2, dtype=torch.float32) + 100 * p for p in range(n)])
    assert torch.equal(a2a, want)
    buf = torch.full((5,), float(me))
    baselines.broadcast(buf, n - 1)
    assert torch.all(buf == n - 1)
    dist.barrier()
    dist.destroy_process_group()


def ep_collective_baseline():
    """The all-to-all (torch.distributed) baseline of dispatch / combine against the reference routing, and a
    round trip with identity experts against the de-quantised input."""
    import torch.distributed as dist
    from rocshmem_b200.baselines.ep import NcclEpDispatcher
    from rocshmem_b200.ops import moe
    dist.init_process_group("gloo", rank=RANK, world_size=WORLD)
    me, P = RANK, WORLD
    E, K, H = 4 * P, 3, 256
    d = NcclEpDispatcher(E, K, H)
    for rep in range(2):
        routing = [moe.make_routing(37 + r, E, K, seed=10 * rep + r) for r in range(P)]
        if rep == 1:
            for idx, _ in routing:
                idx[::4, -1] = -1
        xs = [torch.randn(37 + r, H, generator=torch.Generator().manual_seed(100 * rep + r)).to(torch.bfloat16)
              for r in range(P)]
        idx, w = routing[me]
        res = d.dispatch(xs[me], idx, w)
        want_rows = moe.ref_dispatch([r[0] for r in routing], P, E)[me]
        assert sum(res.recv_counts) == len(want_rows) == res.recv_x.shape[0]
        pos = 0
        epr = E // P
        for s in range(P):
            mine = [t for ss, t in want_rows if ss == s]
            assert res.recv_counts[s] == len(mine)
            rows = slice(pos, pos + len(mine))
            pos += len(mine)
            if not mine:
                continue
            assert res.src_token[rows].tolist() == mine
            q, sc = moe.ref_quantize_1x128(xs[s][mine])
            assert torch.equal(res.recv_x[rows].view(torch.uint8), q.view(torch.uint8))
            assert torch.allclose(res.recv_scales[rows], sc)
            src_idx, src_w = routing[s]
            want_local = torch.where(src_idx[mine] // epr == me, src_idx[mine] % epr, torch.full_like(src_idx[mine], -1))
            want_local = torch.where(src_idx[mine] >= 0, want_local, torch.full_like(want_local, -1))
            assert torch.equal(res.local_expert_idx[rows], want_local.to(torch.int32))
            assert torch.equal(res.gate_weights[rows], src_w[mine])
        y = moe.ref_dequantize_1x128(res.recv_x, res.recv_scales).to(torch.bfloat16)
        out = d.combine(y, idx, w, xs[me].shape[0])
        q, sc = moe.ref_quantize_1x128(xs[me])
        deq = moe.ref_dequantize_1x128(q, sc).to(torch.bfloat16).float()
        gates = torch.where(idx >= 0, w, torch.zeros_like(w)).sum(dim=1, keepdim=True)
        assert torch.allclose(out.float(), deq * gates, rtol=2e-2, atol=2e-2)
    assert d.collectives == 2 * 5
    dist.barrier()
    dist.destroy_process_group()


def data_parallel():
    """Gradient buckets over the world team: averaged gradients of a small model against the gradient of the mean
    loss over all ranks' batches, with buckets small enough to need several, mixed dtypes and an unused parameter."""
    from rocshmem_b200.parallel.data_parallel import GradientBuckets
    init("32M")
    me, n = shm.my_pe(), shm.n_pes()

    def make_model():
        torch.manual_seed(5)
        m = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Tanh(), torch.nn.Linear(40, 17), torch.nn.Tanh(),
                                torch.nn.Linear(17, 3))
        m.extra = torch.nn.Parameter(torch.ones(5))                          # never used: no gradient
        m.scale = torch.nn.Parameter(torch.ones(3, dtype=torch.bfloat16))    # another dtype: its own bucket
        return m

    def batch(r, step):
        g = torch.Generator().manual_seed(1000 * step + r)
        return torch.randn(8, 24, generator=g), torch.randn(8, 3, generator=g)

    def loss_of(m, x, y):
        return ((m(x) * m.scale.float() - y) ** 2).mean()

    used_before = shm.heap_info()["used"]
    model = make_model().to(dev())     # on the CUDA backend the model lives on the GPU (stream-ordered kernels)
    dp = GradientBuckets(list(model.parameters()), bucket_bytes=2048)
    assert len(dp.buckets) >= 3
    for step in range(3):
        model.zero_grad(set_to_none=True)
        x, y = batch(me, step)
        loss_of(model, x.to(dev()), y.to(dev())).backward()
        dp.finish()
        ref = make_model()
        for r in range(n):
            xr, yr = batch(r, step)
            (loss_of(ref, xr, yr) / n).backward()
        for (name, p), q in zip(model.named_parameters(), ref.parameters()):
            want = q.grad if q.grad is not None else torch.zeros_like(q)
            tol = 2e-2 if p.dtype == torch.bfloat16 else (1e-4 if shm.is_cuda() else 1e-5)
            assert torch.allclose(p.grad.float().cpu(), want.float(), rtol=tol, atol=tol), (step, name)
    # without hooks: everything is packed and reduced in finish()
    dp.destroy()
    dp = GradientBuckets(list(model.parameters()), bucket_bytes=1 << 20, average=False, register_hooks=False)
    model.zero_grad(set_to_none=True)
    x, y = batch(me, 9)
    loss_of(model, x.to(dev()), y.to(dev())).backward()
    mine = model[0].weight.grad.clone()
    dp.finish()
    total = shm.zeros(mine.numel(), torch.float32)
    part = shm.zeros(mine.numel(), torch.float32)
    part.copy_(mine.reshape(-1))
    assert coll.reduce(total, part, shm.OP_SUM) == 0
    assert torch.allclose(model[0].weight.grad.reshape(-1).cpu(), total.cpu(), rtol=1e-5, atol=1e-6)
    shm.free(part)
    shm.free(total)
    dp.destroy()
    assert shm.heap_info()["used"] == used_before
    shm.finalize()


def ulysses():
    """Sequence-parallel attention through the all-to-all re-sharding: every rank holds a slice of the sequence,
    attention runs per head on whole sequences, the result comes back as sequence slices and must equal the
    single-process computation."""
    from rocshmem_b200.parallel.ulysses import UlyssesResharder
    init("32M")
    me, n = shm.my_pe(), shm.n_pes()
    S, H, D = 8 * n, 2 * n, 16
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(S, H, D, generator=g) for _ in range(3))
    used_before = shm.heap_info()["used"]
    sp = UlyssesResharder(S, H, D, torch.float32)
    sl, hl = S // n, H // n
    mine = slice(me * sl, (me + 1) * sl)
    qh, kh, vh = (sp.seq_to_heads(t[mine].contiguous().to(dev())) for t in (q, k, v))
    heads = slice(me * hl, (me + 1) * hl)
    assert torch.equal(qh.cpu(), q[:, heads]) and torch.equal(kh.cpu(), k[:, heads]) and torch.equal(vh.cpu(), v[:, heads])

    def attention(q_, k_, v_):                   # [S, h, D] per head, causal
        scores = torch.einsum("shd,thd->hst", q_, k_) / D ** 0.5
        scores = scores.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        return torch.einsum("hst,thd->shd", torch.softmax(scores, dim=-1), v_)

    o_heads = attention(qh.cpu(), kh.cpu(), vh.cpu())
    o_seq = sp.heads_to_seq(o_heads.contiguous().to(dev()))
    want = attention(q, k, v)[mine]
    assert torch.allclose(o_seq.cpu(), want, rtol=1e-5, atol=1e-6)
    try:
        sp.seq_to_heads(torch.zeros(sl + 1, H, D).to(dev()))
        raise AssertionError("a wrong shape must be refused")
    except ValueError:
        pass
    sp.destroy()
    assert shm.heap_info()["used"] == used_before
    shm.finalize()


def ring_attention():
    """Context parallelism: keys and values travel around the ring (put, counter, wait), every rank accumulates its
    queries' attention online; the result equals single-process attention, causal and not."""
    from rocshmem_b200.parallel.ring import RingExchange, ring_attention as ring_attn
    init("32M")
    me, n = shm.my_pe(), shm.n_pes()
    S, H, D = 6 * n, 3, 8
    sl = S // n
    g = torch.Generator().manual_seed(17)
    q, k, v = (torch.randn(S, H, D, generator=g) for _ in range(3))
    mine = slice(me * sl, (me + 1) * sl)
    used_before = shm.heap_info()["used"]
    rk, rv = RingExchange((sl, H, D), torch.float32), RingExchange((sl, H, D), torch.float32)
    # the exchange by itself: after j shifts everybody holds the block of the rank j to its left
    blk = torch.full((sl, H, D), float(me)).to(dev())
    for j in range(1, 2 * n + 1):
        blk = rk.shift(blk)
        assert torch.all(blk.cpu() == float((me - j) % n)), (j, blk.flatten()[:2])
    rk.destroy()
    rk = RingExchange((sl, H, D), torch.float32)

    def full(causal):
        scores = torch.einsum("shd,thd->hst", q, k) / D ** 0.5
        if causal:
            scores = scores.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        return torch.einsum("hst,thd->shd", torch.softmax(scores, dim=-1), v)

    for causal in (False, True):
        out = ring_attn(q[mine].to(dev()), k[mine].to(dev()), v[mine].to(dev()), rk, rv, causal=causal)
        assert torch.allclose(out.cpu(), full(causal)[mine], rtol=1e-5, atol=1e-5), causal
        shm.barrier_all()
    rk.destroy()
    rv.destroy()
    assert shm.heap_info()["used"] == used_before
    shm.finalize()


def pipeline_stages():
    """Three pipeline stages with the all-forward, all-backward schedule: losses and parameter gradients equal
    those of the whole model run in one process over the same micro-batches."""
    from rocshmem_b200.parallel.pipeline import PipelineStage
    init("32M")
    me, n = shm.my_pe(), shm.n_pes()
    d, mb, micro = 12, 4, 5

    def make_layers():
        torch.manual_seed(21)
        return [torch.nn.Sequential(torch.nn.Linear(d, d), torch.nn.Tanh()) for _ in range(n)]

    g = torch.Generator().manual_seed(4)
    xs = [torch.randn(mb, d, generator=g) for _ in range(micro)]
    ys = [torch.randn(mb, d, generator=g) for _ in range(micro)]
    loss_fn = lambda out, tgt: ((out - tgt) ** 2).mean()
    used_before = shm.heap_info()["used"]
    mine = make_layers()[me].to(dev())
    xs_dev, ys_dev = [x.to(dev()) for x in xs], [y.to(dev()) for y in ys]
    stage = PipelineStage(mine, num_stages=n, act_shape=(mb, d))
    assert stage.active and stage.stage == me
    for rep in range(2):
        mine.zero_grad(set_to_none=True)
        losses = stage.run(micro_batches=xs_dev if me == 0 else None, loss_fn=loss_fn if me == n - 1 else None,
                           targets=ys_dev if me == n - 1 else None, num_micro=micro)
        ref = make_layers()
        ref_losses = []
        for x, y in zip(xs, ys):
            h = x
            for layer in ref:
                h = layer(h)
            l = loss_fn(h, y)
            l.backward()
            ref_losses.append(l.detach())
        tol = 1e-4 if shm.is_cuda() else 1e-5
        for p, q in zip(mine.parameters(), ref[me].parameters()):
            assert torch.allclose(p.grad.cpu(), q.grad, rtol=tol, atol=tol / 10), rep
        if me == n - 1:
            assert torch.allclose(torch.stack(losses).cpu(), torch.stack(ref_losses), rtol=tol, atol=tol / 10)
        else:
            assert losses is None
        shm.barrier_all()
    stage.destroy()
    assert shm.heap_info()["used"] == used_before
    shm.finalize()


def alltoallv_host():
    """Variable-count all-to-all: random counts (zeros included), rows tagged with source, destination and index."""
    from rocshmem_b200.ops.host_algorithms import HostAllToAllV
    init("32M")
    me, n = shm.my_pe(), shm.n_pes()
    a2av = HostAllToAllV()
    W = 6
    for rep in range(3):
        gen = torch.Generator().manual_seed(77 + rep)
        counts = torch.randint(0, 9, (n, n), generator=gen)          # counts[s, d], known to everybody for the check
        if rep == 1:
            counts[:, 0] = 0                                         # nobody sends to PE 0
        send = counts[me]
        src = shm.zeros((int(counts.sum(dim=1).max()), W), torch.int32)
        dst = shm.zeros((int(counts.sum(dim=0).max()), W), torch.int32)
        rows = []
        for d in range(n):
            for i in range(int(send[d])):
                rows.append([me, d, i, rep, 0, 0])
        if rows:
            src[:len(rows)] = torch.tensor(rows, dtype=torch.int32).to(dev())
        recv = a2av(dst, src, send.tolist())
        assert recv.tolist() == counts[:, me].tolist()
        got = dst.cpu()[:int(recv.sum())].tolist()
        want = [[s, me, i, rep, 0, 0] for s in range(n) for i in range(int(counts[s, me]))]
        assert got == want, (rep, got[:3], want[:3])
        shm.barrier_all()
        shm.free(dst)
        shm.free(src)
    # a destination that is too small is refused on every PE alike
    src = shm.zeros((8, W), torch.int32)
    dst = shm.zeros((3, W), torch.int32)
    try:
        a2av(dst, src, [1] * n)
        raise AssertionError("an overflowing exchange must be refused")
    except ValueError:
        pass
    shm.barrier_all()
    a2av.destroy()
    shm.finalize()


def elastic_shrink():
    """Rank 2 of 4 leaves between two steps; the others rebuild a world of three (not a strided subset of the old
    one), restore their heap tensors from a snapshot and go on with collectives."""
    from rocshmem_b200.parallel.elastic import shrink
    from rocshmem_b200.parallel.membership import Membership
    from rocshmem_b200.utils import checkpoint
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    assert n == 4
    mem = Membership(shm.runtime.bootstrap_store(), me, n, prefix="elastic")
    weights = shm.zeros(32, torch.float64)
    total = shm.zeros(32, torch.float64)
    weights.copy_((torch.arange(32, dtype=torch.float64) + 100 * me).to(dev()))
    assert coll.reduce(total, weights, shm.OP_SUM) == 0
    assert torch.equal(total.cpu(), torch.arange(32, dtype=torch.float64) * 4 + 100 * 6)
    saved = checkpoint.snapshot({"weights": weights})
    result = shrink(mem, leaving=(me == 2))
    if me == 2:
        assert result is None and not shm.is_initialized()
        print("rank 2 left", flush=True)
        return
    new_pe, new_n = result
    assert new_n == 3 and new_pe == {0: 0, 1: 1, 3: 2}[me]
    assert shm.my_pe() == new_pe and shm.n_pes() == 3
    weights = shm.zeros(32, torch.float64)
    total = shm.zeros(32, torch.float64)
    checkpoint.restore({"weights": weights}, saved)
    assert coll.reduce(total, weights, shm.OP_SUM) == 0
    assert torch.equal(total.cpu(), torch.arange(32, dtype=torch.float64) * 3 + 100 * (0 + 1 + 3))
    # point-to-point with the new numbering: old rank 3 is now PE 2
    probe = shm.zeros(1, torch.int64)
    shm.barrier_all()
    shm.putmem(probe, torch.tensor([me + 10]).to(dev()), (new_pe + 1) % 3)
    shm.barrier_all()
    assert int(probe.cpu()[0]) == {0: 3, 1: 0, 2: 1}[new_pe] + 10
    shm.barrier_all()
    shm.finalize()


def elastic_unplanned():
    """A rank disappears between two steps without a word; the others notice that its heartbeat went stale, record
    it as gone, rebuild a world of two and go on."""
    import time
    from rocshmem_b200.parallel.elastic import shrink
    from rocshmem_b200.parallel.membership import Membership
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    assert n == 3
    mem = Membership(shm.runtime.bootstrap_store(), me, n, prefix="unplanned")
    x = shm.zeros(4, torch.int64)
    y = shm.zeros(4, torch.int64)
    x.fill_(me + 1)
    assert coll.reduce(y, x) == 0 and int(y.cpu()[0]) == 6
    shm.barrier_all()
    if me == 1:
        os._exit(0)                                # gone: no leave record, no finalize
    deadline = time.time() + 30
    stale = []
    while time.time() < deadline:
        mem.heartbeat()
        stale = mem.stale(3.0)
        if stale:
            break
        time.sleep(0.1)
    assert stale == [1], stale
    new_pe, new_n = shrink(mem, dead=stale)
    assert (new_pe, new_n) == ({0: 0, 2: 1}[me], 2)
    x = shm.zeros(4, torch.int64)
    y = shm.zeros(4, torch.int64)
    x.fill_(me + 1)
    assert coll.reduce(y, x) == 0 and int(y.cpu()[0]) == 1 + 3
    shm.barrier_all()
    shm.finalize()


def reduce_scatter_host():
    """Reduce-scatter over the world and over a strided team, every operation and three element types, against
    torch."""
    init("16M")
    me, n = shm.my_pe(), shm.n_pes()
    blk = 6
    world = shm.team_world()
    evens = world.split_strided(0, 2, (n + 1) // 2)
    types = (torch.float32, torch.int64, torch.bfloat16)
    src_w = {dt: shm.zeros(n * blk, dt) for dt in types}
    dst_w = {dt: shm.zeros(blk, dt) for dt in types}
    ops = ((shm.OP_SUM, lambda a: a.sum(0)), (shm.OP_MAX, lambda a: a.max(0).values),
           (shm.OP_MIN, lambda a: a.min(0).values), (shm.OP_PROD, lambda a: a.prod(0)))
    for team, members in ((world, list(range(n))), (evens, list(range(0, n, 2)))):
        m = len(members)
        for dtype in types:
            # small integers: sums and products of up to n of them are exact in every type
            data = {r: ((torch.arange(m * blk) % 5) - 2 + (r % 2)).to(dtype) for r in range(n)}
            src, dst = src_w[dtype], dst_w[dtype]
            src[:m * blk].copy_(data[me].to(dev()))
            shm.barrier_all()
            if me in members:
                i = members.index(me)
                stack = torch.stack([data[r] for r in members])
                wide = stack.double() if dtype.is_floating_point else stack.long()
                for op, fn in ops:
                    assert coll.reduce_scatter(dst, src[:m * blk], op, team) == 0
                    want = fn(wide)[i * blk:(i + 1) * blk].to(dtype)
                    assert torch.equal(dst.cpu(), want), (dtype, op, dst.cpu(), want)
            shm.barrier_all()
    if evens.valid:
        evens.destroy()
    shm.barrier_all()
    shm.finalize()


def elastic_grow():
    """Two ranks run; a third process joins between two steps and the world becomes three."""
    import datetime
    import torch.distributed as dist
    from rocshmem_b200.parallel import elastic
    timeout = float(os.environ.get("ROCSHMEM_TEST_TIMEOUT", "60"))
    if RANK < 2:
        shm.init(rank=RANK, world_size=2, heap_size="16M", backend=BACKEND, timeout_s=timeout)
        x, y = shm.zeros(4, torch.int64), shm.zeros(4, torch.int64)
        x.fill_(RANK + 1)
        assert coll.reduce(y, x) == 0 and int(y.cpu()[0]) == 3
        shm.barrier_all()
        pe, n = elastic.grow(3)
        assert (pe, n) == (RANK, 3)
    else:
        store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), 3, False,
                              timeout=datetime.timedelta(seconds=timeout))
        pe, n = elastic.join(store, 2, timeout_s=timeout, heap_size="16M", backend=BACKEND)
        assert (pe, n) == (2, 3)
    assert shm.my_pe() == RANK and shm.n_pes() == 3
    x, y = shm.zeros(4, torch.int64), shm.zeros(4, torch.int64)
    x.fill_(RANK + 1)
    assert coll.reduce(y, x) == 0 and int(y.cpu()[0]) == 6
    shm.putmem(x, torch.full((4,), 40 + RANK, dtype=torch.int64).to(dev()), (RANK + 1) % 3)
    shm.barrier_all()
    assert int(x.cpu()[0]) == 40 + (RANK - 1) % 3
    shm.barrier_all()
    shm.finalize()


SCENARIOS = {f.__name__: f for f in (elastic_grow, reduce_scatter_host, elastic_unplanned, elastic_shrink, alltoallv_host, pipeline_stages, ring_attention, ulysses, data_parallel, ep_collective_baseline, collective_baselines, threads_host, host_algorithms, stress_host, parallel_layout, moe_layer_host, ep_host, proxy_collectives, host_plumbing, store_bootstrap, teams, team_multicast_standin, collectives_host, wait_and_signal,
                                     late_rank, rank_leaves, team_member_leaves)}

if __name__ == "__main__":
    name = sys.argv[1]
    if name.startswith("gpu_"):
        import mp_gpu_scenarios
        mp_gpu_scenarios.SCENARIOS[name]()
    else:
        SCENARIOS[name]()
    print(f"rank {RANK}: {name} ok")
