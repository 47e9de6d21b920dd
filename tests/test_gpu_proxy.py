"""Reverse-offload path on the GPU (ROCSHMEM_USE_PROXY=1): thread-scope puts, gets and atomics issued by device
code are written as commands into the pinned-host ring and executed by the host proxy thread, which completes
them while the kernel waits (reference: src/reverse_offload/context_ro_device.cpp:457-664, backend_ro.cpp:281-294)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NPES = 2
RMA_PUT, RMA_GET = 0, 2
SC_THREAD = 0
A_FADD, A_FINC, A_ADD, A_INC, A_FCSWAP, A_FETCH, A_SET, A_SWAP, A_FAND, A_AND, A_FOR, A_OR, A_FXOR, A_XOR = range(14)
PROXY_CMD = 28  # ROCSHMEM_STAT_PROXY_CMD


@pytest.fixture(scope="module")
def env():
    import rocshmem_b200 as shm
    from rocshmem_b200 import _native
    if shm.is_initialized():
        shm.finalize()
    shm.init(n_local=NPES, heap_size="64M", ROCSHMEM_WAIT_TIMEOUT_MS=5000, ROCSHMEM_USE_PROXY=1)
    yield shm, _native.load_test_kernels()
    torch.cuda.synchronize()
    shm.finalize()


def test_device_rma_and_atomics_through_the_ring(env):
    from rocshmem_b200 import runtime as rt
    shm, k = env
    C = rt._C()
    assert C.proxy_running()
    side = torch.cuda.Stream()   # the kernel waits for the host thread, which works on streams of its own
    nbytes, threads = 2048, 8
    src = shm.zeros(nbytes, torch.uint8)
    dst = shm.zeros(nbytes, torch.uint8)
    pats = []
    for l in range(NPES):
        p = torch.randint(0, 256, (nbytes,), generator=torch.Generator().manual_seed(5 + l), dtype=torch.uint8)
        pats.append(p)
        shm.local_view(src, l).copy_(p.cuda())
    torch.cuda.synchronize()
    shm.barrier_all()
    C.reset_stats()
    for op, origin in ((RMA_PUT, lambda l: (l - 1) % NPES), (RMA_GET, lambda l: (l + 1) % NPES)):
        for l in range(NPES):
            shm.local_view(dst, l).zero_()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            k.rma(op, SC_THREAD, dst.data_ptr(), src.data_ptr(), nbytes, 1, 0, threads, side.cuda_stream)
        torch.cuda.synchronize()
        err = shm.get_error()
        assert err["count"] == 0, err
        for l in range(NPES):
            assert torch.equal(shm.local_view(dst, l).cpu(), pats[origin(l)]), (op, l)
    executed = C.host_stats()[PROXY_CMD]
    assert executed >= 2 * NPES * threads, executed     # every thread's put and get went through the host
    for t in (dst, src):
        shm.free(t)


def test_device_atomics_through_the_ring_single_pe():
    """Fetching atomics executed by the host thread while the kernel waits for the fetched value. One PE per
    process here: the host's helper kernel has to run next to the waiting kernel, which a cooperative launch
    (several PEs per process) does not allow."""
    import rocshmem_b200 as shm
    from rocshmem_b200 import _native, runtime as rt
    if shm.is_initialized():
        shm.finalize()
    shm.init(n_local=1, heap_size="64M", ROCSHMEM_WAIT_TIMEOUT_MS=5000, ROCSHMEM_USE_PROXY=1)
    try:
        k = _native.load_test_kernels()
        assert rt._C().proxy_running()
        side = torch.cuda.Stream()
        threads, iters = 8, 3
        msgs = threads * iters
        target = shm.zeros(1, torch.int64)
        ret = shm.zeros(threads, torch.int64)
        before = rt._C().host_stats()[PROXY_CMD]
        # Every atomic family goes through the ring (the reference's reverse-offload backend routes all of them
        # through the host, src/reverse_offload/context_ro_tmpl_device.hpp:210-275); oracles as in the direct test.
        for test in range(14):
            target.zero_()
            ret.zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                k.amo(test, target.data_ptr(), ret.data_ptr(), iters, 1, threads, side.cuda_stream)
            torch.cuda.synchronize()
            err = shm.get_error()
            assert err["count"] == 0, (test, err)
            final, best = int(target.cpu()[0]), int(ret.max().cpu())
            want = {A_FADD: (2 * msgs, 2 * (msgs - 1)), A_FINC: (msgs, msgs - 1), A_ADD: (2 * msgs, 0),
                    A_INC: (msgs, 0), A_FCSWAP: (msgs, msgs - 1), A_FETCH: (0, 0), A_SET: (44, 0), A_SWAP: (1, 1),
                    A_FAND: (0, 0), A_AND: (0, 0), A_FOR: (0xFFFF, 0xFFFF), A_OR: (0xFFFF, 0),
                    A_FXOR: (0xFFFF if msgs % 2 else 0, 0xFFFF), A_XOR: (0xFFFF if msgs % 2 else 0, 0)}[test]
            assert (final, best) == want, (test, final, best, want)
        assert rt._C().host_stats()[PROXY_CMD] - before >= 14 * msgs, "the atomics did not go through the ring"
        # put with signal: the payload is stored directly (the one PE is its own neighbour), the signal is a command.
        nbytes = 64 * 128
        src, dst = shm.zeros(nbytes, torch.uint8), shm.zeros(nbytes, torch.uint8)
        sig, fetched = shm.zeros(1, torch.int64), shm.zeros(2, torch.int64)
        src.fill_(ord("7"))
        for sig_op, start, expect in ((0, 123, 1), (1, 123, 123 + 64)):
            sig.fill_(start)
            dst.zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                k.signal(SC_THREAD, sig_op, dst.data_ptr(), src.data_ptr(), nbytes, sig.data_ptr(), 1, expect,
                         fetched.data_ptr(), 64, side.cuda_stream)
            torch.cuda.synchronize()
            err = shm.get_error()
            assert err["count"] == 0, (sig_op, err)
            assert int(sig.cpu()[0]) == expect and fetched.cpu().tolist() == [expect, 0]
            assert torch.all(dst.cpu() == ord("7"))
    finally:
        torch.cuda.synchronize()
        shm.finalize()


STAT_PROXY_SLOT_NS, STAT_PROXY_PACK_NS, STAT_PROXY_HOST_NS, STAT_WAIT_NS = 30, 31, 32, 33


def _fresh(**kw):
    import rocshmem_b200 as shm
    from rocshmem_b200 import _native
    if shm.is_initialized():
        shm.finalize()
    shm.init(heap_size="64M", ROCSHMEM_WAIT_TIMEOUT_MS=5000, **kw)
    return shm, _native.load_test_kernels()


def test_warp_coalescing_merges_proxied_puts_and_gets_and_time_buckets_fill():
    from rocshmem_b200 import runtime as rt
    shm, k = _fresh(n_local=2, ROCSHMEM_USE_PROXY=1, ROCSHMEM_USE_WF_COAL=1)
    try:
        C = rt._C()
        side = torch.cuda.Stream()
        nbytes, threads = 4096, 32
        src = shm.zeros(nbytes, torch.uint8)
        dst = shm.zeros(nbytes, torch.uint8)
        pats = []
        for l in range(2):
            p = torch.randint(0, 256, (nbytes,), generator=torch.Generator().manual_seed(5 + l), dtype=torch.uint8)
            pats.append(p)
            shm.local_view(src, l).copy_(p.cuda())
        torch.cuda.synchronize()
        shm.barrier_all()
        C.reset_stats()
        before = C.host_stats()[28]
        for op, origin in ((RMA_PUT, lambda l: (l - 1) % 2), (RMA_GET, lambda l: (l + 1) % 2)):
            for l in range(2):
                shm.local_view(dst, l).zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                k.rma(op, SC_THREAD, dst.data_ptr(), src.data_ptr(), nbytes, 1, 0, threads, side.cuda_stream)
            torch.cuda.synchronize()
            assert shm.get_error()["count"] == 0
            for l in range(2):
                assert torch.equal(shm.local_view(dst, l).cpu(), pats[origin(l)]), (op, l)
        executed = C.host_stats()[28] - before
        # 32 lanes with adjacent equal shares: one command per warp and operation instead of 32
        assert executed <= 2 * 2 * 2, executed
        for l in range(2):
            st = C.device_stats(l)
            assert st[STAT_PROXY_PACK_NS] > 0 and st[STAT_PROXY_HOST_NS] > 0, st[28:34]
    finally:
        torch.cuda.synchronize()
        shm.finalize()
