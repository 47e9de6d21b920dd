"""The slab (bump) allocator carved out of the symmetric heap (reference: SlabHeap / DevMonoLinear,
src/memory/slab_heap.cpp:31-114, dev_mono_linear.hpp:41-140). Host-side half on the CPU backend; the device
half shares the placement arithmetic (`detail::slab_place`)."""
import torch

from rocshmem_b200 import runtime as rt


def test_slab_hands_out_aligned_increasing_blocks_until_exhausted(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=2, heap_size="4M", backend="host", ROCSHMEM_SLAB_SIZE="8K")
    C = rt._C()
    try:
        base, size = C.slab_create(0)                # size from ROCSHMEM_SLAB_SIZE
        assert base != 0 and size == 8192 and base % 128 == 0
        a = C.slab_alloc_host(base, size, 100, 16)
        b = C.slab_alloc_host(base, size, 1, 1)
        c = C.slab_alloc_host(base, size, 64, 256)
        assert a == base and b == base + 100 and c == base + 256
        assert C.slab_used(base, size) == 256 + 64
        assert C.slab_alloc_host(base, size, 0, 16) == 0              # empty request
        assert C.slab_alloc_host(base, size, 8, 3) == 0               # alignment not a power of two
        assert C.slab_alloc_host(base, size, 8192, 16) == 0           # does not fit ...
        assert C.slab_used(base, size) == 320                         # ... and leaves the cursor alone
        d = C.slab_alloc_host(base, size, 8192 - 320, 1)              # exactly the rest
        assert d == base + 320 and C.slab_used(base, size) == 8192
        assert C.slab_alloc_host(base, size, 1, 1) == 0
        C.slab_reset(base, size)
        assert C.slab_used(base, size) == 0 and C.slab_alloc_host(base, size, 8, 8) == base
        # the slab is an ordinary symmetric object: a second one does not overlap it, and freeing works
        base2, size2 = C.slab_create(1000)
        assert size2 == 1024 and (base2 >= base + size + 256 or base2 + size2 + 256 <= base)
        C.slab_destroy(base2, size2)
        C.slab_destroy(base, size)
        # larger than the heap: reported, not fatal
        assert C.slab_create(1 << 30)[0] == 0
    finally:
        shm.finalize()


def test_slab_memory_is_usable_by_rma(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=2, heap_size="4M", backend="host")
    C = rt._C()
    try:
        base, size = C.slab_create(4096)
        p = C.slab_alloc_host(base, size, 64 * 8, 128)
        src = shm.zeros(64, torch.int64)
        src.copy_(torch.arange(64) + 5)
        C.putmem(p, src.data_ptr(), 64 * 8, 1)       # same offset inside PE 1's slab
        got = shm.zeros(64, torch.int64)
        C.getmem(got.data_ptr(), p, 64 * 8, 1)
        assert torch.equal(shm.local_view(got, 0), torch.arange(64) + 5)
        C.slab_destroy(base, size)
    finally:
        shm.finalize()
