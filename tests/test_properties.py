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


# ---- host RMA and atomics against a model -----------------------------------------------------------------------------

_RMA_OP = st.one_of(
    st.tuples(st.just("put"), st.integers(0, 3), st.integers(0, 3), st.integers(0, 63), st.integers(0, 63),
              st.integers(1, 64)),                                   # origin PE, target PE, source offset, dest offset, n
    st.tuples(st.just("get"), st.integers(0, 3), st.integers(0, 3), st.integers(0, 63), st.integers(0, 63),
              st.integers(1, 64)),
    st.tuples(st.just("fadd"), st.integers(0, 3), st.integers(0, 3), st.integers(0, 127), st.integers(-50, 50),
              st.just(0)),                                           # origin, target, index, value
    st.tuples(st.just("swap"), st.integers(0, 3), st.integers(0, 3), st.integers(0, 127), st.integers(-50, 50),
              st.just(0)),
    st.tuples(st.just("cas"), st.integers(0, 3), st.integers(0, 3), st.integers(0, 127), st.integers(-3, 3),
              st.integers(-3, 3)),                                   # origin, target, index, compare, value
)


@settings(max_examples=25, deadline=None)
@given(st.lists(_RMA_OP, min_size=1, max_size=60))
def test_host_rma_and_atomics_match_a_model(ops):
    """Random sequences of puts, gets and atomics between four PEs of one process (CPU backend) against plain
    Python lists: every returned value and the final content of every PE's array."""
    import torch

    import rocshmem_b200 as shm
    if shm.is_initialized():
        shm.finalize()
    shm.init(n_local=4, heap_size="4M", backend="host")
    try:
        N = 128
        arr = shm.zeros(N, torch.int64)
        model = [[0] * N for _ in range(4)]
        for pe in range(4):
            init = [(pe + 1) * 1000 + i for i in range(N)]
            shm.local_view(arr, pe).copy_(torch.tensor(init))
            model[pe] = init
        for op, origin, target, a, b, c in ops:
            shm.set_local_pe(origin)
            mine = shm.local_view(arr, origin)
            if op == "put":
                n = min(c, N - a, N - b)
                shm.putmem(mine[b:b + n], mine[a:a + n].clone(), target)     # dest offset b on the target
                model[target][b:b + n] = model[origin][a:a + n]
            elif op == "get":
                n = min(c, N - a, N - b)
                tmp = torch.zeros(n, dtype=torch.int64)
                shm.getmem(tmp, mine[a:a + n], target)                       # source offset a on the target
                assert tmp.tolist() == model[target][a:a + n]
                shm.local_view(arr, origin)[b:b + n] = tmp
                model[origin][b:b + n] = model[target][a:a + n]
            elif op == "fadd":
                old = shm.atomic_fetch_add(mine, b, target, index=a)
                assert old == model[target][a]
                model[target][a] += b
            elif op == "swap":
                old = shm.atomic_swap(mine, b, target, index=a)
                assert old == model[target][a]
                model[target][a] = b
            else:
                # make the comparison hit now and then: values near zero only occur after swaps
                old = shm.atomic_compare_swap(mine, b, c, target, index=a)
                assert old == model[target][a]
                if model[target][a] == b:
                    model[target][a] = c
        shm.set_local_pe(0)
        shm.quiet()
        for pe in range(4):
            assert shm.local_view(arr, pe).tolist() == model[pe], pe
    finally:
        shm.set_local_pe(0)
        shm.finalize()


# ---- host collectives on random strided teams against torch ---------------------------------------------------------------

@settings(max_examples=20, deadline=None)
@given(st.integers(0, 7), st.integers(1, 4), st.integers(1, 8), st.integers(1, 70),
       st.sampled_from(["int32", "int64", "float32", "float64", "bfloat16", "int16"]),
       st.sampled_from(["sum", "min", "max", "prod", "and", "or", "xor"]), st.integers(0, 10 ** 6))
def test_host_collectives_on_random_teams_match_torch(start, stride, size, nelems, dtype_name, op_name, seed):
    """Eight PEs in one process (CPU backend): a random strided team, then reduce, broadcast, fcollect and alltoall
    on it against the same operations computed with torch; PEs outside the team keep their buffers."""
    import torch

    import rocshmem_b200 as shm
    from rocshmem_b200.ops import collectives as coll
    P = 8
    if start + (size - 1) * stride >= P:
        size = (P - 1 - start) // stride + 1
    dtype = getattr(torch, dtype_name)
    if op_name in ("and", "or", "xor") and dtype.is_floating_point:
        op_name = "max"
    op = {"sum": shm.OP_SUM, "min": shm.OP_MIN, "max": shm.OP_MAX, "prod": shm.OP_PROD, "and": shm.OP_AND,
          "or": shm.OP_OR, "xor": shm.OP_XOR}[op_name]
    if shm.is_initialized():
        shm.finalize()
    shm.init(n_local=P, heap_size="4M", backend="host")
    try:
        members = [start + i * stride for i in range(size)]
        team = shm.team_world().split_strided(start, stride, size)
        g = torch.Generator().manual_seed(seed)
        src = shm.zeros(nelems * size, dtype)
        dst = shm.zeros(nelems * size, dtype)
        data = []
        for pe in range(P):
            # small integers: products of up to eight of them stay exact in every type, bf16 included
            v = torch.randint(-2, 3, (nelems * size,), generator=g).to(dtype)
            data.append(v)
            shm.local_view(src, pe).copy_(v)
            shm.local_view(dst, pe).fill_(7)
        # reduce
        assert coll.reduce(dst[:nelems], src[:nelems], op, team) == 0
        stack = torch.stack([data[m][:nelems] for m in members])
        wide = stack.double() if dtype.is_floating_point else stack.long()
        want = {"sum": lambda: wide.sum(0), "min": lambda: wide.min(0).values, "max": lambda: wide.max(0).values,
                "prod": lambda: wide.prod(0)}.get(op_name)
        if want is None:
            acc = wide[0].clone()
            for row in wide[1:]:
                acc = {"and": acc & row, "or": acc | row, "xor": acc ^ row}[op_name]
            expect = acc
        else:
            expect = want()
        for pe in range(P):
            got = shm.local_view(dst, pe)[:nelems]
            if pe in members:
                assert torch.equal(got.double() if dtype.is_floating_point else got.long(), expect.to(got.device)), (pe, op_name)
            else:
                assert torch.all(got == 7)
        # broadcast from the last member: everybody but the root receives
        root = size - 1
        for pe in range(P):
            shm.local_view(dst, pe).fill_(7)
        assert coll.broadcast(dst[:nelems], src[:nelems], root, team) == 0
        for i, m in enumerate(members):
            got = shm.local_view(dst, m)[:nelems]
            assert torch.equal(got, data[members[root]][:nelems]) if i != root else torch.all(got == 7)
        # fcollect and alltoall
        assert coll.fcollect(dst, src[:nelems], team) == 0
        for m in members:
            got = shm.local_view(dst, m).view(size, nelems)
            assert all(torch.equal(got[i], data[members[i]][:nelems]) for i in range(size))
        assert coll.alltoall(dst, src, team) == 0
        for j, m in enumerate(members):
            got = shm.local_view(dst, m).view(size, nelems)
            assert all(torch.equal(got[i], data[members[i]].view(size, nelems)[j]) for i in range(size))
        team.destroy()
    finally:
        shm.set_local_pe(0)
        shm.finalize()
