"""Device half of the slab (bump) allocator: threads, warps and blocks of a kernel allocate from a slab carved out
of the symmetric heap (reference: SlabHeap / DevMonoLinear, src/memory/slab_heap.cpp:31-114,
dev_mono_linear.hpp:41-140). The host half and the shared placement arithmetic are covered in test_slab.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _fresh(**kw):
    import rocshmem_b200 as shm
    from rocshmem_b200 import _native
    if shm.is_initialized():
        shm.finalize()
    shm.init(heap_size="64M", ROCSHMEM_WAIT_TIMEOUT_MS=5000, **kw)
    return shm, _native.load_test_kernels()


def test_slab_allocation_from_kernels():
    from rocshmem_b200 import runtime as rt
    shm, k = _fresh()
    try:
        C = rt._C()
        blocks, threads, each = 4, 128, 48
        base, size = C.slab_create(1 << 20)
        n = blocks * threads
        tp = torch.zeros(n, dtype=torch.int64, device="cuda")
        wp = torch.zeros(n // 32, dtype=torch.int64, device="cuda")
        bp = torch.zeros(blocks, dtype=torch.int64, device="cuda")
        errors = torch.zeros(1, dtype=torch.int32, device="cuda")
        k.slab_test(base, size, each, tp.data_ptr(), wp.data_ptr(), bp.data_ptr(), errors.data_ptr(), blocks, threads,
                    torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert int(errors.item()) == 0
        spans = [(p, each) for p in tp.tolist()] + [(p, 64) for p in wp.tolist()] + [(p, 256) for p in bp.tolist()]
        assert all(base <= p and p + s <= base + size for p, s in spans)
        assert all(p % 16 == 0 for p in tp.tolist()) and all(p % 64 == 0 for p in wp.tolist())
        assert all(p % 256 == 0 for p in bp.tolist())
        spans.sort()
        assert all(a + s <= b for (a, s), (b, _) in zip(spans, spans[1:])), "allocations overlap"
        assert C.slab_used(base, size) >= n * each + (n // 32) * 64 + blocks * 256
        # exhaustion: requests that do not fit return null and leave the cursor alone
        C.slab_reset(base, size)
        used0 = C.slab_used(base, size)
        k.slab_test(base, size, size, tp.data_ptr(), wp.data_ptr(), bp.data_ptr(), errors.data_ptr(), 1, 32,
                    torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        got = tp[:32].tolist()
        assert sum(1 for p in got if p != 0) == 1 and used0 == 0      # exactly one thread gets the whole slab
        C.slab_destroy(base, size)
    finally:
        torch.cuda.synchronize()
        shm.finalize()
