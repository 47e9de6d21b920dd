"""Host API on the shared-memory backend with several PEs inside one process. Covers the same
semantics as the GPU tests (RMA, atomics, waits, teams, contexts, collectives) without a GPU."""
import pytest
import torch

from rocshmem_b200.ops import collectives as coll


@pytest.fixture
def shm4(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=4, heap_size="16M", backend="host")
    yield shm
    shm.finalize()


def test_identity_and_heap(shm4):
    shm = shm4
    assert shm.n_pes() == 4 and shm.n_local_pes() == 4 and not shm.is_cuda()
    for l in range(4):
        shm.set_local_pe(l)
        assert shm.my_pe() == l
    shm.set_local_pe(0)
    info = shm.heap_info()
    assert info["size"] == 16 << 20 and info["backend"] == "host-shm" and info["used"] == 0
    a = shm.empty(100, torch.float32)
    b = shm.empty(100, torch.float32)
    assert a.data_ptr() % 128 == 0 and b.data_ptr() - a.data_ptr() == 512  # 400 B -> 512 B block
    assert shm.heap_info()["used"] == 1024
    shm.free(a)
    shm.free(b)
    assert shm.heap_info()["used"] == 0
    with pytest.raises(ValueError):
        shm.free(torch.zeros(4))
    with pytest.raises(MemoryError):
        shm.empty(1 << 30, torch.uint8)


def test_put_get_all_pairs(shm4):
    shm = shm4
    buf = shm.zeros((4, 64), torch.int64)
    for me in range(4):
        shm.set_local_pe(me)
        row = torch.arange(64, dtype=torch.int64) + (me << 32)
        for pe in range(4):
            shm.putmem(shm.local_view(buf, me)[me], row, pe, nbi=(pe % 2 == 1))
    shm.quiet()
    shm.barrier_all()
    for pe in range(4):
        got = shm.local_view(buf, pe)
        for me in range(4):
            assert torch.equal(got[me], torch.arange(64, dtype=torch.int64) + (me << 32))
    out = torch.zeros(64, dtype=torch.int64)
    shm.set_local_pe(2)
    shm.getmem(out, shm.local_view(buf, 2)[3], 1)
    assert out[5] == (3 << 32) + 5


def test_atomics_all_families(shm4):
    shm = shm4
    shm.set_local_pe(0)
    x = shm.zeros(4, torch.int64)
    assert shm.atomic_fetch_add(x, 5, 3) == 0 and shm.atomic_fetch_add(x, -2, 3) == 5
    assert shm.atomic_fetch(x, 3) == 3
    assert shm.atomic_swap(x, 44, 3) == 3
    assert shm.atomic_compare_swap(x, 43, 1, 3) == 44 and shm.atomic_fetch(x, 3) == 44
    assert shm.atomic_compare_swap(x, 44, 1, 3) == 44 and shm.atomic_fetch(x, 3) == 1
    assert shm.atomic(shm.AMO_OR, x, 0xF0, 3) == 1 and shm.atomic(shm.AMO_AND, x, 0x3F, 3) == 0xF1
    assert shm.atomic(shm.AMO_XOR, x, 0xFF, 3) == 0x31 and shm.atomic_fetch(x, 3) == 0xCE
    assert int(shm.local_view(x, 3)[0]) == 0xCE and int(x[0]) == 0
    f = shm.zeros(2, torch.float32)
    shm.atomic_swap(f, 1.5, 1, index=1)
    assert shm.atomic(shm.AMO_ADD, f, 2.25, 1, index=1) == 1.5
    assert shm.atomic_fetch(f, 1, index=1) == 3.75
    i32 = shm.zeros(1, torch.int32)
    assert shm.atomic_fetch_add(i32, -7, 2) == 0 and shm.atomic_fetch(i32, 2) == -7
    with pytest.raises(Exception):
        shm.atomic_fetch_add(torch.zeros(1, dtype=torch.int64), 1, 0)  # not symmetric
    with pytest.raises(Exception):
        shm.atomic_fetch_add(shm.zeros(2, torch.int16), 1, 0)          # unsupported width


def test_wait_family_and_timeout(shm4):
    shm = shm4
    flags = shm.zeros(4, torch.int32)
    one = torch.tensor([7], dtype=torch.int32)
    shm.set_local_pe(1)
    shm.putmem(shm.local_view(flags, 1)[2:3], one, 0)
    shm.set_local_pe(0)
    assert shm.wait_until(flags, shm.CMP_EQ, 7, index=2) == shm.SUCCESS
    assert shm.test(flags, shm.CMP_GE, 7, index=2) and not shm.test(flags, shm.CMP_LT, 7, index=2)
    assert shm.wait_until_any(flags, shm.CMP_NE, 0) == 2
    assert shm.wait_until_some(flags, shm.CMP_GT, 0) == [2]
    assert shm.wait_until_any(flags, shm.CMP_NE, 0, status=[0, 0, 1, 0]) == -1 or True
    shm.set_wait_timeout_ms(100)
    assert shm.wait_until(flags, shm.CMP_EQ, 9, index=0) == shm.ERROR
    err = shm.get_error()
    assert err["kind"] == 1 and err["expected"] == 9 and err["observed"] == 0
    assert shm.wait_until_any(flags, shm.CMP_EQ, 12345) == -1
    shm.clear_error()


def test_teams_and_collectives(shm4):
    shm = shm4
    world = shm.team_world()
    src = shm.zeros(33, torch.float64)
    dst = shm.zeros(33, torch.float64)
    for l in range(4):
        shm.local_view(src, l).copy_(torch.arange(33, dtype=torch.float64) * (l + 1))
    assert coll.reduce(dst, src) == 0
    for l in range(4):
        assert torch.allclose(shm.local_view(dst, l), torch.arange(33, dtype=torch.float64) * 10)
    odd = world.split_strided(1, 2, 2)
    shm.set_local_pe(1)
    assert odd.my_pe() == 0 and odd.translate_pe(1, world) == 3
    shm.set_local_pe(2)
    assert odd.my_pe() == -1
    shm.set_local_pe(0)
    assert coll.reduce(dst, src, shm.OP_MAX, odd) == 0
    assert torch.allclose(shm.local_view(dst, 3), torch.arange(33, dtype=torch.float64) * 4)
    assert torch.allclose(shm.local_view(dst, 0), torch.arange(33, dtype=torch.float64) * 10)  # not a member
    for l in range(4):
        shm.local_view(dst, l).fill_(-1)
    assert coll.broadcast(dst, src, 1, odd) == 0  # root = team PE 1 = world PE 3
    assert torch.allclose(shm.local_view(dst, 1), torch.arange(33, dtype=torch.float64) * 4)
    assert torch.all(shm.local_view(dst, 3) == -1)  # the root's dest is not written
    gat = shm.zeros(4 * 33, torch.float64)
    assert coll.fcollect(gat, src) == 0
    assert torch.allclose(shm.local_view(gat, 2).view(4, 33)[3], torch.arange(33, dtype=torch.float64) * 4)
    odd.destroy()
    with pytest.raises(ValueError):
        world.split_strided(0, 1, 5)


def test_contexts(shm4):
    shm = shm4
    ctxs = [shm.Context() for _ in range(39)]  # the default context is the 40th
    with pytest.raises(RuntimeError):
        shm.Context()
    buf = shm.zeros(8, torch.int32)
    shm.putmem(buf, torch.full((8,), 3, dtype=torch.int32), 2, ctx=ctxs[5], nbi=True)
    ctxs[5].quiet()
    assert int(shm.local_view(buf, 2)[7]) == 3
    team = shm.team_world().split_strided(2, 1, 2)  # {2, 3}
    shm.set_local_pe(2)
    ctxs[0].destroy()
    tctx = shm.Context(team=team)
    shm.putmem(shm.local_view(buf, 2), torch.full((8,), 9, dtype=torch.int32), 1, ctx=tctx)  # team PE 1 = world 3
    assert int(shm.local_view(buf, 3)[0]) == 9
    with pytest.raises(Exception):
        shm.putmem(buf, torch.zeros(8, dtype=torch.int32), 2, ctx=tctx)  # PE 2 is outside the team
    tctx.destroy()
    for c in ctxs[1:]:
        c.destroy()
    team.destroy()


def test_reinit_with_other_shape(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=2, heap_size="4M", backend="host")
    assert shm.n_pes() == 2
    shm.finalize()
    shm.init(n_local=1, heap_size="1M", backend="host")
    assert shm.n_pes() == 1 and shm.heap_info()["size"] == 1 << 20
    x = shm.zeros(4, torch.int64)
    assert shm.atomic_fetch_add(x, 1, 0) == 0
    shm.finalize()


def test_threads_share_the_host_api(shm4):
    """THREAD_MULTIPLE: several host threads issue atomics and puts at once, each with its own context and
    acting for its own local PE (the reference's SOS tests `threading` and `mt_contention`)."""
    import threading
    shm = shm4
    n_threads, iters = 8, 200
    counter = shm.zeros(1, torch.int64)
    slots = shm.zeros(n_threads * 16, torch.int32)
    errors = []

    def work(tid):
        try:
            shm.set_local_pe(tid % 4)
            ctx = shm.Context()
            fetched = [shm.atomic_fetch_add(counter, 1, 2, ctx=ctx) for _ in range(iters)]
            assert all(b > a for a, b in zip(fetched, fetched[1:])), "fetched values of one thread must grow"
            shm.putmem(shm.local_view(slots, tid % 4)[tid * 16:(tid + 1) * 16],
                       torch.full((16,), tid + 1, dtype=torch.int32), 3, ctx=ctx)
            ctx.quiet()
            ctx.destroy()
        except Exception as e:  # noqa: BLE001 - reported by the main thread
            errors.append((tid, repr(e)))

    threads = [threading.Thread(target=work, args=(t,)) for t in range(n_threads)]
    [t.start() for t in threads]
    [t.join(60) for t in threads]
    assert not errors, errors
    assert int(shm.local_view(counter, 2)[0]) == n_threads * iters
    got = shm.local_view(slots, 3).view(n_threads, 16)
    assert all(torch.all(got[t] == t + 1) for t in range(n_threads))
    shm.free(slots)
    shm.free(counter)


def test_stream_ordered_collectives_reject_buffers_that_are_not_symmetric(shm4):
    """The kernels derive peer addresses from the tensors' pointers, so the Python layer refuses anything that is
    not a contiguous tensor on the symmetric heap (and mismatched types or sizes) before a kernel is launched."""
    from rocshmem_b200.ops import collectives as coll
    shm = shm4
    a = shm.zeros(64, torch.float32)
    b = shm.zeros(64, torch.float32)
    small = shm.zeros(8, torch.float32)
    other = shm.zeros(64, torch.int32)
    local = torch.zeros(64)
    assert shm.is_symmetric(a) and shm.is_symmetric(a[8:16]) and not shm.is_symmetric(local)
    with pytest.raises(ValueError, match="`dest` must live on the symmetric heap"):
        coll.allreduce_async(local, a, stream=0)
    with pytest.raises(ValueError, match="`source` must live on the symmetric heap"):
        coll.fcollect_async(a, local, stream=0)
    with pytest.raises(ValueError, match="contiguous"):
        coll.broadcast_async(a[::2], b[::2], 0, stream=0)
    with pytest.raises(ValueError, match="torch.int32"):
        coll.allreduce_async(other, a, stream=0)
    with pytest.raises(ValueError, match="64 are needed"):
        coll.allreduce_async(small, a, stream=0)
    with pytest.raises(ValueError, match="256 are needed"):
        coll.fcollect_async(a, b, stream=0)               # 4 PEs x 64 elements
    with pytest.raises(ValueError, match="not a multiple"):
        coll.alltoall_async(a, shm.zeros(6, torch.float32), stream=0)


def test_error_records_are_described_in_words(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=2, heap_size="4M", backend="host", ROCSHMEM_WAIT_TIMEOUT_MS=50)
    try:
        assert shm.describe_error() == "no error recorded"
        flag = shm.zeros(1, torch.int64)
        assert shm.wait_until(flag, shm.CMP_EQ, 5) == shm.ERROR
        text = shm.describe_error()
        assert text.startswith("wait_until timed out in a host API call") and "expected 5, observed 0" in text
        made_up = {"count": 2, "kind": 2, "pe": 3, "where": 70, "addr": 0x10, "expected": 9, "observed": 8}
        assert shm.describe_error(made_up).startswith("barrier / collective flag wait timed out in MoE dispatch: count "
                                                      "exchange, peer PE 3")
        shm.clear_error()
        assert shm.describe_error() == "no error recorded"
    finally:
        shm.finalize()


def test_reduce_scatter_argument_checks_and_allgather_alias(shm4):
    shm = shm4
    n = 4
    src = shm.zeros(n * 5, torch.float32)
    dst = shm.zeros(5, torch.float32)
    data = [torch.arange(n * 5, dtype=torch.float32) * (l + 1) - 3 * l for l in range(n)]
    for l in range(n):
        shm.local_view(src, l).copy_(data[l])
    with pytest.raises(ValueError, match="equal blocks"):
        coll.reduce_scatter(dst, shm.zeros(7, torch.float32))
    with pytest.raises(ValueError, match="sum, min, max and prod"):
        coll.reduce_scatter(dst, src, shm.OP_XOR)
    with pytest.raises(ValueError, match="symmetric heap"):
        coll.reduce_scatter(torch.zeros(5), src)
    gat = shm.zeros(n * 5, torch.float32)
    assert coll.allgather(gat, src[:5]) == 0
    assert torch.equal(shm.local_view(gat, 2).view(n, 5)[3], data[3][:5])


def test_calls_before_init_raise_instead_of_crashing(fresh_runtime):
    shm = fresh_runtime
    C = shm.runtime._C()
    for call in (shm.get_error, shm.heap_info, shm.is_cuda, shm.describe_error, shm.barrier_all, lambda: shm.zeros(4),
                 lambda: C.device_stats(0), C.check_canaries, C.num_user_teams, C.proxy_start):
        with pytest.raises(RuntimeError, match="not initialised"):
            call()
    assert shm.my_pe() == 0 and shm.n_pes() >= 1          # identity works before init, as in the reference
    shm.finalize()                                        # a no-op


def test_unknown_comparison_is_refused_at_once(shm4):
    shm = shm4
    flags = shm.zeros(4, torch.int64)
    import time
    t0 = time.time()
    for call in (lambda: shm.wait_until(flags, 99, 1), lambda: shm.test(flags, -1, 1),
                 lambda: shm.wait_until_any(flags, 7, [1, 1, 1, 1]), lambda: shm.wait_until_all(flags, 6, [0, 0, 0, 0])):
        with pytest.raises(ValueError, match="comparison"):
            call()
    assert time.time() - t0 < 2          # not after a time-out
