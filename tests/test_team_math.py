"""Team arithmetic: split validation and PE translation (reference: src/team.cpp:51-111,
src/rocshmem.cpp:221-303; SOS test shmem_team_translate)."""
from rocshmem_b200 import _native

C = _native.load()
WORLD8 = (0, 1, 8)


def test_split_of_world():
    assert C.plan_split(0, 1, 8, 8, 0, 2, 4) == (0, 2, 4)
    assert C.plan_split(0, 1, 8, 8, 1, 3, 3) == (1, 3, 3)
    assert C.plan_split(0, 1, 8, 8, 7, 1, 1) == (7, 1, 1)


def test_split_rejections():
    for start, stride, size in ((-1, 1, 1), (8, 1, 1), (0, 0, 2), (0, 1, 0), (0, 1, 9), (0, 2, 5), (4, 1, 5), (1, 7, 3)):
        assert C.plan_split(0, 1, 8, 8, start, stride, size) is None, (start, stride, size)


def test_nested_split_composes_strides():
    # parent = {1, 3, 5, 7}; child takes parent PEs 1 and 3 -> world 3 and 7
    assert C.plan_split(1, 2, 4, 8, 1, 2, 2) == (3, 4, 2)
    assert C.plan_split(1, 2, 4, 8, 0, 1, 4) == (1, 2, 4)
    assert C.plan_split(1, 2, 4, 8, 2, 2, 2) is None  # parent PE 4 does not exist


def test_translate():
    even, odd = (0, 2, 4), (1, 2, 4)
    assert C.translate_pe(even, 3, WORLD8) == 6
    assert C.translate_pe(WORLD8, 6, even) == 3
    assert C.translate_pe(WORLD8, 5, even) == -1
    assert C.translate_pe(even, 1, odd) == -1
    assert C.translate_pe(even, 4, WORLD8) == -1 and C.translate_pe(even, -1, WORLD8) == -1
    quad = (0, 4, 2)
    assert C.translate_pe(even, 2, quad) == 1 and C.translate_pe(quad, 1, even) == 2


def test_lowest_common_slot():
    assert C.lowest_common_slot([0b1110, 0b1100, 0b1111]) == 2
    assert C.lowest_common_slot([0b0001, 0b0010]) == -1
    assert C.lowest_common_slot([1 << 39]) == 39
