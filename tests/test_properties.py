"""Property tests (hypothesis) of the allocator and the team arithmetic against simple Python models."""
from hypothesis import given, settings, strategies as st

from rocshmem_b200 import _native

C = _native.load()


@settings(max_examples=60, deadline=None)
@given(st.integers(min_value=12, max_value=22),
       st.lists(st.tuples(st.booleans(), st.integers(min_value=1, max_value=1 << 16)), min_size=1, max_size=200))
def test_allocator_invariants(log_size, ops):
    """Whatever the sequence of allocations and frees: blocks are power-of-two sized, aligned to their size up to the
    alignment of their top-level chunk, disjoint, accounted for in used(), and everything merges back at the end."""
    size = (1 << log_size) + 384          # not a power of two
    a = C.Pow2Allocator(size)
    live = {}
    for do_alloc, n in ops:
        if do_alloc or not live:
            off = a.alloc(n)
            if off is None:
                assert n > a.largest_free_block()
                continue
            blk = a.block_size(off)
            assert blk >= max(n, 128) and blk & (blk - 1) == 0 and off % 128 == 0 and off + blk <= size
            assert blk < 2 * max(n, 128)
            for o, b in live.items():
                assert off + blk <= o or o + b <= off
            live[off] = blk
        else:
            off = sorted(live)[n % len(live)]
            assert a.free(off) and not a.free(off)
            del live[off]
        assert a.used() == sum(live.values()) and a.live_allocations() == len(live)
    for off in list(live):
        assert a.free(off)
    assert a.used() == 0 and a.largest_free_block() == 1 << log_size


def members(triplet):
    start, stride, size = triplet
    return [start + stride * i for i in range(size)]


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 64), st.integers(0, 63), st.integers(1, 8), st.integers(1, 64),
       st.integers(-1, 64), st.integers(0, 8), st.integers(0, 64))
def test_split_matches_a_set_model(world, p_start, p_stride, p_size, start, stride, size):
    """plan_split accepts exactly the requests whose members exist in the parent, and the new team is the parent's
    members at positions start, start + stride, ..."""
    parent = (p_start, p_stride, p_size)
    if p_start + p_stride * (p_size - 1) >= world:
        return                                        # not a valid parent in this world
    got = C.plan_split(p_start, p_stride, p_size, world, start, stride, size)
    pm = members(parent)
    positions = [start + stride * i for i in range(size)] if stride >= 1 and size >= 1 else []
    valid = bool(positions) and start >= 0 and all(0 <= q < p_size for q in positions)
    if not valid:
        assert got is None
        return
    assert got is not None
    assert members(got) == [pm[q] for q in positions]
    # translation between the new team and the world is consistent with membership
    for i, w in enumerate(members(got)):
        assert C.translate_pe(got, i, (0, 1, world)) == w
        assert C.translate_pe((0, 1, world), w, got) == i
    outside = [w for w in range(world) if w not in members(got)]
    for w in outside[:5]:
        assert C.translate_pe((0, 1, world), w, got) == -1
