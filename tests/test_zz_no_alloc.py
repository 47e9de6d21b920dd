"""The allocation-free expert-layout entry point, called through its exported C symbol.

Some users of this library may not allocate device memory when they need the expert layout: an
inference server that gave all GPU memory to its own pool at start-up, a plug-in inside such a server,
or a latency path where an allocation could stall the device. For them the shared library exports
``rocshmem_b200_expert_layout_noalloc`` (declared in ``csrc/kernels/no_alloc.h``), which keeps its
per-expert cursors in a fixed array inside the library. This test runs a real MoE dispatch, asks both
the regular entry point (caller-provided scratch) and the new one for the layout, and expects the same
answer: identical offsets, and per expert the same set of (row, k) pairs (the order inside one expert's
range is unspecified for both). It does so twice in a row with different routings, because the fixed
scratch keeps the previous call's contents.

The file name sorts after the other test files so that it is collected last.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -2
BAD_ARGUMENT = -3


@pytest.fixture(scope="module")
def shm():
    import rocshmem_b200 as s
    if s.is_initialized():
        s.finalize()
    s.init(n_local=1, heap_size="1G", ROCSHMEM_WAIT_TIMEOUT_MS=5000)
    yield s
    torch.cuda.synchronize()
    s.finalize()


@pytest.fixture(scope="module")
def entry():
    import rocshmem_b200
    path = os.path.join(os.path.dirname(rocshmem_b200.__file__), "lib", "librocshmem_b200.so")
    lib = ctypes.CDLL(path)
    fn = lib.rocshmem_b200_expert_layout_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def grouped(offsets, row_index, pair_k):
    """Per expert, the sorted list of (row, k) pairs."""
    off = offsets.cpu().tolist()
    rows = row_index[:off[-1]].cpu().tolist()
    ks = pair_k[:off[-1]].cpu().tolist()
    return off, [sorted(zip(rows[a:b], ks[a:b])) for a, b in zip(off[:-1], off[1:])]


def run_both(shm, entry, d, T, H, E, K, seed, out, side_stream=False):
    from rocshmem_b200.ops import moe
    dev = shm.device()
    x = shm.zeros((T, H), torch.bfloat16)
    idx = shm.zeros((T, K), torch.int32)
    w = shm.zeros((T, K), torch.float32)
    il, wl = moe.make_routing(T, E, K, seed)
    il[::7, -1] = -1  # some unused top-k entries
    x.copy_(torch.randn(T, H, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16).to(dev))
    idx.copy_(il.to(dev))
    w.copy_(wl.to(dev))
    d.dispatch(x, idx, w)
    want = grouped(*d.expert_layout())
    offsets, row_index, pair_k = out
    # A stream of the caller's own: the work is ordered after the dispatch, which ran on the current stream.
    side = torch.cuda.Stream() if side_stream else None
    if side is not None:
        side.wait_stream(torch.cuda.current_stream())
    stream = (side or torch.cuda.current_stream()).cuda_stream
    rc = entry(d.recv_meta.data_ptr(), d.recv_info.data_ptr(), 1, E, K, offsets.data_ptr(), row_index.data_ptr(),
               pair_k.data_ptr(), stream)
    assert rc == 0, f"rocshmem_b200_expert_layout_noalloc returned {rc}"
    torch.cuda.synchronize()
    got = grouped(offsets[:E + 1], row_index, pair_k)
    assert got[0] == want[0], "offsets differ"
    assert got[0][-1] == int((il >= 0).sum()), "every routed (token, k) pair has a position"
    assert got[1] == want[1], "per-expert (row, k) sets differ"
    err = shm.get_error(0)
    assert err["count"] == 0, err
    for t in (x, idx, w):
        shm.free(t)


def test_noalloc_matches_regular_entry_point_twice(shm, entry):
    from rocshmem_b200.ops import moe
    T, H, K = 300, 1024, 4
    big, small = 64, 8
    d_big = moe.EpDispatcher(big, K, H, T)
    d_small = moe.EpDispatcher(small, K, H, T)
    # Outputs are the caller's; they are allocated here, before the calls under test.
    out = (torch.empty(big + 1, dtype=torch.int32, device="cuda"),
           torch.empty(T * K, dtype=torch.int32, device="cuda"),
           torch.empty(T * K, dtype=torch.int32, device="cuda"))
    # Two calls in a row on one dispatcher with different routings, then fewer experts (the cursors of
    # the earlier, larger call are still in the library's array), then the larger one again.
    run_both(shm, entry, d_big, T, H, big, K, seed=11, out=out)
    run_both(shm, entry, d_big, T, H, big, K, seed=12, out=out)
    run_both(shm, entry, d_small, T, H, small, K, seed=13, out=out)
    run_both(shm, entry, d_big, T, H, big, K, seed=14, out=out)
    run_both(shm, entry, d_big, T, H, big, K, seed=15, out=out, side_stream=True)


def test_noalloc_rejects_sizes_beyond_its_scratch(shm, entry):
    """More experts per rank than the built-in array holds: refused on the host, nothing is launched."""
    buf = torch.zeros(4096, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    assert entry(p, p, 1, 1025, 4, p, p, p, 0) == TOO_LARGE
    assert entry(p, p, 1, 8, 9, p, p, p, 0) == TOO_LARGE
    assert entry(p, p, 0, 8, 4, p, p, p, 0) == BAD_ARGUMENT
    assert entry(None, p, 1, 8, 4, p, p, p, 0) == BAD_ARGUMENT
    torch.cuda.synchronize()
