"""Device API exercised from user-style kernels on one GPU that hosts several PEs (one cooperative
launch, blockIdx.z selects the PE). Re-expresses the reference's functional test matrix
(scripts/functional_tests/driver.sh: rma / amo / sigops / coll / other groups) with its oracles."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NPES = 4
RMA_PUT, RMA_PUT_NBI, RMA_GET, RMA_GET_NBI, RMA_P, RMA_G = range(6)
SC_THREAD, SC_WARP, SC_BLOCK = range(3)


@pytest.fixture(scope="module")
def env():
    import rocshmem_b200 as shm
    from rocshmem_b200 import _native
    if shm.is_initialized():
        shm.finalize()
    shm.init(n_local=NPES, heap_size="256M", ROCSHMEM_WAIT_TIMEOUT_MS=4000, ROCSHMEM_MAX_NUM_CONTEXTS=48)
    k = _native.load_test_kernels()
    yield shm, k
    torch.cuda.synchronize()
    shm.finalize()


def stream():
    return torch.cuda.current_stream().cuda_stream


def views(shm, t):
    return [shm.local_view(t, l) for l in range(NPES)]


def sync_ok(shm):
    torch.cuda.synchronize()
    err = shm.get_error()
    assert err["count"] == 0, err


def test_backend_is_cuda_vmm(env):
    shm, _ = env
    info = shm.heap_info()
    assert shm.is_cuda() and info["backend"] == "cuda-vmm" and shm.n_pes() == NPES
    assert info["stride"] % (2 << 20) == 0


@pytest.mark.parametrize("scope", [SC_THREAD, SC_WARP, SC_BLOCK])
@pytest.mark.parametrize("op", [RMA_PUT, RMA_PUT_NBI, RMA_GET, RMA_GET_NBI])
@pytest.mark.parametrize("nbytes", [8, 1000, 4096 + 24, 1 << 20])
def test_rma(env, op, scope, nbytes):
    shm, k = env
    src = shm.zeros(nbytes, torch.uint8)
    dst = shm.zeros(nbytes, torch.uint8)
    pats = []
    for l, v in enumerate(views(shm, src)):
        g = torch.Generator(device="cpu").manual_seed(100 + l)
        p = torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8)
        pats.append(p)
        v.copy_(p.cuda())
    torch.cuda.synchronize()
    shm.barrier_all()
    threads = 64 if scope == SC_THREAD else 256
    k.rma(op, scope, dst.data_ptr(), src.data_ptr(), nbytes, 1, int(scope == SC_BLOCK), threads, stream())
    sync_ok(shm)
    for l, v in enumerate(views(shm, dst)):
        # put: PE l's dst was written by PE l-1; get: PE l read from PE l+1
        origin = (l - 1) % NPES if op in (RMA_PUT, RMA_PUT_NBI) else (l + 1) % NPES
        assert torch.equal(v.cpu(), pats[origin]), (op, scope, nbytes, l)
    shm.free(dst)
    shm.free(src)


@pytest.mark.parametrize("op", [RMA_P, RMA_G])
def test_p_and_g(env, op):
    shm, k = env
    n = 512
    src = shm.zeros(n, torch.int64)
    dst = shm.zeros(n, torch.int64)
    for l, v in enumerate(views(shm, src)):
        v.copy_((torch.arange(n) + (l << 32)).cuda())
    torch.cuda.synchronize()
    shm.barrier_all()
    k.rma(op, SC_THREAD, dst.data_ptr(), src.data_ptr(), n * 8, 2, 1, 128, stream())
    sync_ok(shm)
    for l, v in enumerate(views(shm, dst)):
        origin = (l - 2) % NPES if op == RMA_P else (l + 2) % NPES
        assert torch.equal(v.cpu(), torch.arange(n) + (origin << 32))
    shm.free(dst)
    shm.free(src)


A_FADD, A_FINC, A_ADD, A_INC, A_FCSWAP, A_FETCH, A_SET, A_SWAP, A_FAND, A_AND, A_FOR, A_OR, A_FXOR, A_XOR = range(14)


@pytest.mark.parametrize("test", list(range(14)))
def test_atomics_int64(env, test):
    shm, k = env
    blocks, threads, iters = 2, 64, 5
    target = shm.zeros(1, torch.int64)
    ret = shm.zeros(blocks * threads, torch.int64)
    msgs = NPES * blocks * threads * iters
    if test in (A_FAND, A_AND):
        target.fill_(0)  # reference oracle: and / fetch_and of 0xFFFF on 0 stays 0
    torch.cuda.synchronize()
    shm.barrier_all()
    k.amo(test, target.data_ptr(), ret.data_ptr(), iters, blocks, threads, stream())
    sync_ok(shm)
    final = int(target.cpu()[0])
    best = max(int(v.max().cpu()) for v in views(shm, ret))
    if test == A_FADD:
        assert best == 2 * (msgs - 1) and final == 2 * msgs
    elif test == A_FINC:
        assert best == msgs - 1 and final == msgs
    elif test == A_ADD:
        assert final == 2 * msgs
    elif test == A_INC:
        assert final == msgs
    elif test == A_FCSWAP:
        assert final == msgs and best == msgs - 1
    elif test == A_FETCH:
        assert final == 0 and best == 0
    elif test == A_SET:
        assert final == 44
    elif test == A_SWAP:
        assert 1 <= final <= NPES and 0 <= best <= NPES
    elif test in (A_FAND, A_AND):
        assert final == 0
    elif test in (A_FOR, A_OR):
        assert final == 0xFFFF and (test == A_OR or best == 0xFFFF)
    elif test in (A_FXOR, A_XOR):
        assert final == (0xFFFF if msgs % 2 else 0)
    shm.free(ret)
    shm.free(target)


@pytest.mark.parametrize("pe", [0, 3])
def test_atomics_other_types(env, pe):
    import struct
    shm, k = env
    u32 = shm.zeros(1, torch.int32)
    f32 = shm.zeros(1, torch.float32)
    f64 = shm.zeros(1, torch.float64)
    i32 = shm.zeros(1, torch.int32)
    out = shm.zeros(16, torch.int64)
    k.amo_types(u32.data_ptr(), f32.data_ptr(), f64.data_ptr(), i32.data_ptr(), out.data_ptr(), pe, stream())
    sync_ok(shm)
    o = out.cpu().tolist()
    assert o[0:5] == [0, 7, 0xF7, 5, 9]
    assert struct.unpack("f", struct.pack("I", o[5]))[0] == 1.5
    assert struct.unpack("f", struct.pack("I", o[6]))[0] == 2.5
    assert struct.unpack("d", struct.pack("q", o[7]))[0] == 3.25
    assert o[8:12] == [0, -3, -2, 1]
    assert int(shm.local_view(u32, pe).cpu()[0]) == 9 and float(shm.local_view(f32, pe).cpu()[0]) == 2.5
    for t in (out, i32, f64, f32, u32):
        shm.free(t)


@pytest.mark.parametrize("scope,groups", [(SC_THREAD, 64), (SC_WARP, 2), (SC_BLOCK, 1)])
@pytest.mark.parametrize("sig_op", [0, 1])
def test_put_signal(env, scope, groups, sig_op):
    shm, k = env
    nbytes = 64 * 128
    src = shm.zeros(nbytes, torch.uint8)
    dst = shm.zeros(nbytes, torch.uint8)
    sig = shm.zeros(1, torch.int64)
    fetched = shm.zeros(2, torch.int64)
    for l, v in enumerate(views(shm, src)):
        v.fill_(ord("0") + l)
        shm.local_view(sig, l).fill_(l + 123)
    torch.cuda.synchronize()
    shm.barrier_all()
    value = 1
    for l in range(NPES):
        pass
    # SET leaves `value`; ADD adds one per signalling group to the initial value
    if sig_op == 0:
        expects = [1] * NPES
    else:
        expects = [l + 123 + groups for l in range(NPES)]
    # the kernel takes one `expect` for all PEs, so give every PE the same initial value for ADD
    if sig_op == 1:
        for l in range(NPES):
            shm.local_view(sig, l).fill_(123)
        expects = [123 + groups] * NPES
        torch.cuda.synchronize()
    k.signal(scope, sig_op, dst.data_ptr(), src.data_ptr(), nbytes, sig.data_ptr(), value, expects[0],
             fetched.data_ptr(), 64, stream())
    sync_ok(shm)
    for l in range(NPES):
        assert int(shm.local_view(sig, l).cpu()[0]) == expects[l]
        f = shm.local_view(fetched, l).cpu().tolist()
        assert f == [expects[l], 0]
        assert torch.all(shm.local_view(dst, l).cpu() == ord("0") + (l - 1) % NPES)
    for t in (fetched, sig, dst, src):
        shm.free(t)


def test_pingpong_and_pingall(env):
    shm, k = env
    flag = shm.zeros(1, torch.int32)
    ns = shm.zeros(1, torch.int64)
    iters = 200
    k.pingpong(flag.data_ptr(), iters, ns.data_ptr(), stream())
    sync_ok(shm)
    assert int(flag.cpu()[0]) == iters and int(shm.local_view(flag, 1).cpu()[0]) == iters
    assert int(ns.cpu()[0]) > 0
    slots = shm.zeros(NPES, torch.int64)
    result = shm.zeros(8, torch.int64)
    k.pingall(slots.data_ptr(), result.data_ptr(), stream())
    sync_ok(shm)
    for l in range(NPES):
        assert shm.local_view(slots, l).cpu().tolist() == [p + 1 for p in range(NPES)]
        r = shm.local_view(result, l).cpu().tolist()
        assert r[0] == NPES - 1 and r[1] == NPES and r[2] == 1 and r[3] == NPES - 1
        assert r[4] == 1 and r[5] == 0 and r[6] == -1 and r[7] == -1  # SIZE_MAX reads back as -1
    for t in (result, slots, ns, flag):
        shm.free(t)


def test_wait_timeout_reports_and_context_stays_usable(env):
    shm, k = env
    flag = shm.zeros(1, torch.int64)
    status = shm.zeros(1, torch.int32)
    shm.set_wait_timeout_ms(300)
    try:
        k.timeout(flag.data_ptr(), status.data_ptr(), stream())
        torch.cuda.synchronize()
        for l in range(NPES):
            assert int(shm.local_view(status, l).cpu()[0]) == 1  # ROCSHMEM_ERROR
            err = shm.get_error(l)
            assert err["kind"] == 1 and err["expected"] == 12345 and err["count"] >= 1
    finally:
        shm.clear_error()
        shm.set_wait_timeout_ms(4000)
    # the GPU context is intact: a normal kernel still runs
    k.pingpong(shm.zeros(1, torch.int32).data_ptr(), 3, shm.zeros(1, torch.int64).data_ptr(), stream())
    sync_ok(shm)
    shm.free(status)
    shm.free(flag)


def test_team_context_and_translation(env):
    shm, k = env
    world = shm.team_world()
    odd = world.split_strided(1, 2, 2)  # {1, 3}
    slots = shm.zeros(4, torch.int32)
    out = shm.zeros(4, torch.int32)
    k.team_ctx(odd.handle, world.handle, slots.data_ptr(), out.data_ptr(), stream())
    sync_ok(shm)
    for l in range(NPES):
        o = shm.local_view(out, l).cpu().tolist()
        if l % 2 == 0:
            assert o[0] == -2  # not a member
        else:
            assert o == [0, l // 2, 2, l]
            assert shm.local_view(slots, l).cpu().tolist()[:2] == [100, 101]
    odd.destroy()
    shm.free(out)
    shm.free(slots)


def test_device_context_pool_exhaustion(env):
    shm, k = env
    out = shm.zeros(1, torch.int32)
    k.ctx_exhaust(60, out.data_ptr(), stream())  # pool holds 48
    sync_ok(shm)
    assert int(out.cpu()[0]) == 48
    k.ctx_exhaust(10, out.data_ptr(), stream())  # all were returned
    sync_ok(shm)
    assert int(out.cpu()[0]) == 10
    shm.free(out)


C_BCAST, C_FCOLLECT, C_ALLTOALL, C_SUM, C_MIN, C_MAX, C_PROD, C_AND, C_OR, C_XOR = range(10)
TORCH = {"float32": torch.float32, "float64": torch.float64, "int16": torch.int16, "int32": torch.int32,
         "int64": torch.int64, "long": torch.int64, "int8": torch.int8, "float16": torch.float16,
         "bfloat16": torch.bfloat16}


def make_inputs(dtype, n, npes, lo=-40, hi=40):
    outs = []
    for p in range(npes):
        g = torch.Generator().manual_seed(77 + p)
        if dtype.is_floating_point:
            outs.append(torch.randn(n, generator=g, dtype=torch.float64).to(dtype))
        else:
            outs.append(torch.randint(lo, hi, (n,), generator=g, dtype=torch.int64).to(dtype))
    return outs


@pytest.mark.parametrize("dtype", ["float32", "float64", "int16", "int32", "int64", "long", "float16", "bfloat16"])
@pytest.mark.parametrize("n", [1, 7, 1000, 4099])
def test_block_reduce(env, dtype, n):
    shm, k = env
    td = TORCH[dtype]
    src = shm.zeros(n, td)
    dst = shm.zeros(n, td)
    rc = shm.zeros(1, torch.int32)
    ins = make_inputs(td, n, NPES, -3, 4) if not td.is_floating_point else make_inputs(td, n, NPES)
    for l, v in enumerate(views(shm, src)):
        v.copy_(ins[l].cuda())
    torch.cuda.synchronize()
    shm.barrier_all()
    ops = [C_SUM, C_MIN, C_MAX, C_PROD] + ([] if td.is_floating_point else [C_AND, C_OR, C_XOR])
    wide = torch.float64 if td.is_floating_point else torch.int64
    stack = torch.stack([x.to(wide) for x in ins])
    refs = {C_SUM: stack.sum(0), C_MIN: stack.min(0).values, C_MAX: stack.max(0).values, C_PROD: stack.prod(0)}
    if not td.is_floating_point:
        a, o, x = stack[0].clone(), stack[0].clone(), stack[0].clone()
        for s in stack[1:]:
            a, o, x = a & s, o | s, x ^ s
        refs.update({C_AND: a, C_OR: o, C_XOR: x})
    for op in ops:
        k.coll(op, dtype, shm.team_world().handle, dst.data_ptr(), src.data_ptr(), n, 0, 2, rc.data_ptr(), 256, stream())
        sync_ok(shm)
        for l, v in enumerate(views(shm, dst)):
            got = v.cpu().to(wide)
            if td.is_floating_point:
                tol = {torch.float16: 2e-2, torch.bfloat16: 6e-2}.get(td, 1e-5)
                assert torch.allclose(got, refs[op], rtol=tol, atol=tol * 4), (dtype, n, op, l)
            else:
                assert torch.equal(got, refs[op].to(td).to(wide)), (dtype, n, op, l)
        assert int(rc.cpu()[0]) == 0
    for t in (rc, dst, src):
        shm.free(t)


@pytest.mark.parametrize("dtype", ["float32", "float64", "int8", "int16", "int32", "int64", "long"])
@pytest.mark.parametrize("op", [C_BCAST, C_FCOLLECT, C_ALLTOALL])
def test_block_copy_collectives_on_a_team(env, dtype, op):
    shm, k = env
    td = TORCH[dtype]
    n = 301
    team = shm.team_world().split_strided(0, 1, 3)  # PEs 0..2; PE 3 stays out
    tsize = 3
    src = shm.zeros(n * tsize, td)
    dst = shm.zeros(n * tsize, td)
    rc = shm.zeros(1, torch.int32)
    ins = make_inputs(td, n * tsize, NPES, -100, 100)
    for l, (s, d) in enumerate(zip(views(shm, src), views(shm, dst))):
        s.copy_(ins[l].cuda())
        d.fill_(-5)
    torch.cuda.synchronize()
    shm.barrier_all()
    root = 2
    k.coll(op, dtype, team.handle, dst.data_ptr(), src.data_ptr(), n, root, 1, rc.data_ptr(), 128, stream())
    sync_ok(shm)
    for l, v in enumerate(views(shm, dst)):
        got = v.cpu()
        if l == 3:
            assert torch.all(got == -5)
            continue
        if op == C_BCAST:
            if l == root:
                assert torch.all(got == -5)  # the root's dest is left alone
            else:
                assert torch.equal(got[:n], ins[root][:n]) and torch.all(got[n:] == -5)
        elif op == C_FCOLLECT:
            for p in range(tsize):
                assert torch.equal(got[p * n:(p + 1) * n], ins[p][:n])
        else:
            for p in range(tsize):
                assert torch.equal(got[p * n:(p + 1) * n], ins[p][l * n:(l + 1) * n])
    team.destroy()
    for t in (rc, dst, src):
        shm.free(t)


def test_barrier_and_sync_stress(env):
    shm, k = env
    slots = shm.zeros(NPES, torch.int64)
    errors = shm.zeros(1, torch.int32)
    k.barrier_stress(slots.data_ptr(), 300, errors.data_ptr(), 64, stream())
    sync_ok(shm)
    for l in range(NPES):
        assert int(shm.local_view(errors, l).cpu()[0]) == 0
        assert shm.local_view(slots, l).cpu().tolist() == [300] * NPES
    # host barrier interleaved with device barriers shares the epoch
    shm.barrier_all()
    k.barrier_stress(slots.data_ptr(), 5, errors.data_ptr(), 32, stream())
    sync_ok(shm)
    shm.barrier_all()
    shm.free(errors)
    shm.free(slots)


def test_rocshmem_ptr(env):
    shm, k = env
    buf = shm.zeros(16, torch.uint8)
    k.shmem_ptr(buf.data_ptr(), 4, stream())
    sync_ok(shm)
    for l in range(NPES):
        got = shm.local_view(buf, l).cpu()
        assert int(got[4]) == ord("1") + (l - 1) % NPES and int(got[0]) == 0
    shm.free(buf)


@pytest.mark.parametrize("scope", [SC_THREAD, SC_WARP, SC_BLOCK])
def test_copy_every_size_and_alignment(env, scope):
    shm, k = env
    max_len, max_align = 96, 16
    offs_s = [so for so in range(max_align) if so < 4 or (so - 4) % 5 == 0]
    offs_d = [do for do in range(max_align) if do < 4 or (do - 4) % 7 == 0]
    stride = ((max_len + 2 * max_align + 255) // 256) * 256
    cases = (max_len + 1) * len(offs_s) * len(offs_d)
    src = shm.zeros(cases * stride, torch.uint8)
    dst = shm.zeros(cases * stride, torch.uint8)
    g = torch.Generator().manual_seed(5)
    pat = torch.randint(1, 255, (cases * stride,), generator=g, dtype=torch.uint8)
    for v in views(shm, src):
        v.copy_(pat.cuda())
    torch.cuda.synchronize()
    k.copy_align(scope, dst.data_ptr(), src.data_ptr(), max_len, max_align, 96, stream())
    sync_ok(shm)
    got = dst.cpu().view(cases, stride)
    want = torch.zeros_like(got)
    p2 = pat.view(cases, stride)
    c = 0
    for length in range(max_len + 1):
        for so in offs_s:
            for do in offs_d:
                want[c, do:do + length] = p2[c, so:so + length]
                c += 1
    assert torch.equal(got, want)
    shm.free(dst)
    shm.free(src)


def test_api_surface_compiles_and_launches(env):
    shm, k = env
    buf = shm.zeros(64, torch.uint8)
    k.api_surface(buf.data_ptr(), shm.team_world().handle, stream())
    sync_ok(shm)
    shm.free(buf)


def test_host_api_on_device_heap(env):
    """Host-initiated put / get / atomics / waits / collectives against the GPU heap."""
    from rocshmem_b200.ops import collectives as coll
    shm, _ = env
    a = shm.zeros(1000, torch.int64)
    b = shm.zeros(1000, torch.int64)
    for l, v in enumerate(views(shm, a)):
        v.copy_((torch.arange(1000) + (l << 32)).cuda())
    torch.cuda.synchronize()
    shm.set_local_pe(1)
    shm.putmem(shm.local_view(b, 1), shm.local_view(a, 1), 2)
    assert torch.equal(shm.local_view(b, 2).cpu(), torch.arange(1000) + (1 << 32))
    host = torch.zeros(1000, dtype=torch.int64).pin_memory()
    shm.getmem(host, shm.local_view(a, 1), 3)
    assert torch.equal(host, torch.arange(1000) + (3 << 32))
    shm.set_local_pe(0)
    ctr = shm.zeros(2, torch.int64)
    assert [shm.atomic_fetch_add(ctr, 3, 2, index=1) for _ in range(3)] == [0, 3, 6]
    assert shm.atomic_compare_swap(ctr, 9, 100, 2, index=1) == 9
    assert shm.atomic_swap(ctr, -1, 2, index=1) == 100
    assert shm.wait_until(shm.local_view(ctr, 2), shm.CMP_EQ, -1, index=1) == shm.SUCCESS
    assert shm.test(shm.local_view(ctr, 2), shm.CMP_LT, 0, index=1)
    r = shm.zeros(1000, torch.int64)
    assert coll.reduce(r, a) == 0
    want = torch.arange(1000) * NPES + (sum(range(NPES)) << 32)
    for v in views(shm, r):
        assert torch.equal(v.cpu(), want)
    g = shm.zeros(1000 * NPES, torch.int64)
    assert coll.fcollect(g, a) == 0
    assert torch.equal(shm.local_view(g, 2).cpu().view(NPES, 1000)[3], torch.arange(1000) + (3 << 32))
    for t in (g, r, ctr, b, a):
        shm.free(t)


@pytest.mark.parametrize("nbytes,root", [((3 << 20) + 40, 1), ((9 << 20) + 16, 3), (600 << 10, 0)])
def test_large_broadcast_through_relays(env, nbytes, root):
    """Payloads of 512 KiB and more take the relay path (root -> one part per member -> forwarded): every
    member but the root receives the root's bytes, the root's dest keeps its content."""
    from rocshmem_b200.ops import collectives as coll
    shm, _ = env
    src = shm.zeros(nbytes + 16, torch.uint8)
    dst = shm.zeros(nbytes + 16, torch.uint8)
    pattern = (torch.arange(nbytes, dtype=torch.int64) * 2654435761 >> 7).to(torch.uint8)
    for l, v in enumerate(views(shm, src)):
        v[8:8 + nbytes].copy_(((pattern.to(torch.int32) + l) % 256).to(torch.uint8).cuda())
    for v in views(shm, dst):
        v.fill_(7)
    torch.cuda.synchronize()
    for rep in range(2):
        assert coll.broadcast(dst[8:8 + nbytes], src[8:8 + nbytes], root) == 0
        want = ((pattern.to(torch.int32) + root) % 256).to(torch.uint8)
        for l, v in enumerate(views(shm, dst)):
            got = v.cpu()
            assert torch.all(got[:8] == 7) and torch.all(got[8 + nbytes:] == 7), "wrote outside the range"
            if l == root:
                assert torch.all(got[8:8 + nbytes] == 7), "the root's dest must stay untouched"
            else:
                assert torch.equal(got[8:8 + nbytes], want), (l, rep)
    err = shm.get_error(0)
    assert err["count"] == 0, err
    shm.free(dst)
    shm.free(src)


def test_device_locks_and_grid_sync(env):
    """Ticket lock (per block), spin lock (per thread) and the grid barrier of the rocshmemx extensions:
    increments of a plain counter under each lock must all survive."""
    shm, k = env
    blocks, threads, rounds = 96, 128, 50   # 96 blocks are resident together on a B200 (grid barrier)
    state = torch.zeros(64, dtype=torch.int64, device="cuda")
    errs = torch.zeros(1, dtype=torch.int32, device="cuda")
    base = state.data_ptr()
    k.mutex_test(base, base + 64, base + 128, base + 256, rounds, errs.data_ptr(), blocks, threads,
                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = state.cpu()
    assert int(got[16]) == blocks * rounds, "ticket lock lost updates"
    assert int(got[17]) == blocks * rounds, "spin lock lost updates"
    assert int(got[32]) == blocks, "grid barrier counter"
    assert int(errs.item()) == 0
    assert shm.get_error(0)["count"] == 0


def test_device_statistics_count_api_calls(env):
    """Kernels built with -DROCSHMEM_PROFILE count their API calls per PE (reference: src/stats.hpp);
    reset_stats() zeroes them, device_stats() reads them back."""
    from rocshmem_b200 import runtime as rt
    shm, k = env
    C = rt._C()
    nbytes = 4096
    src = shm.zeros(nbytes, torch.uint8)
    dst = shm.zeros(nbytes, torch.uint8)
    torch.cuda.synchronize()
    C.reset_stats()
    assert sum(C.device_stats(0)) == 0
    threads = 64
    k.rma(RMA_PUT, SC_THREAD, dst.data_ptr(), src.data_ptr(), nbytes, 1, 0, threads, stream())
    sync_ok(shm)
    for l in range(NPES):
        st = C.device_stats(l)
        assert st[0] == threads, (l, st[:8])            # ROCSHMEM_STAT_PUT: one put per thread
        assert st[26] == nbytes, (l, st[24:30])         # ROCSHMEM_STAT_BYTES_PUT
    C.reset_stats()
    assert sum(C.device_stats(1)) == 0
    C.dump_stats()                                        # prints, must not fail
    shm.free(dst)
    shm.free(src)
