"""Symmetric-heap allocator. Mirrors the reference's allocator unit tests
(tests/unit_tests: address_record, bin, binner, pow2_bins, single_heap gtests): bin layout, pow2
rounding, splitting, exhaustion, determinism, plus the buddy merging this implementation adds."""
import random

import pytest

from rocshmem_b200 import _native

C = _native.load()


def test_rounding_and_alignment():
    a = C.Pow2Allocator(1 << 20)
    o1 = a.alloc(1)
    assert o1 == 0 and a.block_size(o1) == 128
    o2 = a.alloc(129)
    assert o2 % 128 == 0 and a.block_size(o2) == 256
    o3 = a.alloc(4096)
    assert a.block_size(o3) == 4096 and o3 % 4096 == 0
    assert a.used() == 128 + 256 + 4096


def test_zero_and_exhaustion_return_none():
    a = C.Pow2Allocator(1 << 12)
    assert a.alloc(0) is None
    assert a.alloc((1 << 12) + 1) is None
    o = a.alloc(1 << 12)
    assert o == 0
    assert a.alloc(1) is None
    assert a.free(o)
    assert a.alloc(1) == 0


def test_non_power_of_two_heap_is_chopped_greedily():
    size = (1 << 20) + (1 << 14) + 128 + 64  # the 64-byte tail is below the alignment
    a = C.Pow2Allocator(size)
    assert a.managed() == size - 64
    assert a.bin_population(1 << 20) == 1 and a.bin_population(1 << 14) == 1 and a.bin_population(128) == 1
    assert a.largest_free_block() == 1 << 20
    big = a.alloc(1 << 20)
    assert big == 0
    assert a.alloc(1 << 15) is None  # only the 16 KiB and 128 B chunks are left
    assert a.alloc(1 << 14) == 1 << 20


def test_split_populates_smaller_bins():
    a = C.Pow2Allocator(1 << 16)
    o = a.alloc(128)
    assert o == 0
    for k in range(7, 16):
        assert a.bin_population(1 << k) == 1, k
    assert a.bin_population(1 << 16) == 0


def test_free_merges_buddies_back():
    a = C.Pow2Allocator(1 << 16)
    offs = [a.alloc(128) for _ in range(512)]
    assert offs == [i * 128 for i in range(512)]
    assert a.alloc(1) is None
    for o in offs:
        assert a.free(o)
    assert a.used() == 0 and a.largest_free_block() == 1 << 16 and a.live_allocations() == 0


def test_double_free_and_foreign_offsets_are_rejected():
    a = C.Pow2Allocator(1 << 16)
    o = a.alloc(1000)
    assert a.free(o) and not a.free(o) and not a.free(12345)


def test_determinism_across_instances():
    rng = random.Random(7)
    script = []
    live = []
    for _ in range(2000):
        if live and rng.random() < 0.45:
            script.append(("f", live.pop(rng.randrange(len(live)))))
        else:
            script.append(("a", rng.choice([1, 100, 128, 129, 4000, 70000, 1 << 20])))
            live.append(len([s for s in script if s[0] == "a"]) - 1)
    def run():
        a = C.Pow2Allocator((1 << 26) + (1 << 20))
        offsets, out = [], []
        for kind, v in script:
            if kind == "a":
                o = a.alloc(v)
                offsets.append(o)
                out.append(o)
            else:
                o = offsets[v]
                out.append(a.free(o) if o is not None else None)
        return out, a.used()
    assert run() == run()


def test_no_overlap_under_random_load():
    rng = random.Random(3)
    a = C.Pow2Allocator(1 << 22)
    live = {}
    for _ in range(5000):
        if live and rng.random() < 0.5:
            o = rng.choice(list(live))
            assert a.free(o)
            del live[o]
        else:
            n = rng.choice([1, 64, 128, 300, 5000, 60000])
            o = a.alloc(n)
            if o is not None:
                size = a.block_size(o)
                assert size >= n and o % 128 == 0
                for p, s in live.items():
                    assert o + size <= p or p + s <= o, "overlap"
                live[o] = size
    assert a.used() == sum(live.values())


def test_bad_alignment_rejected():
    with pytest.raises(Exception):
        C.Pow2Allocator(1 << 20, 100)
