"""Message coalescing of the reverse-offload path (reference: WfCoalOn::coalesce, src/wf_coal_policy.cpp:57-172):
the lane-mask arithmetic that the warp form uses, the list form, and the ring consumer that executes a run of
commands as one transfer. All on the CPU backend."""
import random

import torch

from rocshmem_b200 import runtime as rt


def _plan(active, msgs):
    return rt._C().coalesce_warp_plan(active, msgs)


def _brute(active, msgs):
    """Lane by lane: a lane leads a run that extends over the following active lanes while each continues the
    one before it."""
    lanes = [l for l in range(32) if active >> l & 1]
    runs = [0] * 32
    i = 0
    while i < len(lanes):
        j = i + 1
        while j < len(lanes):
            a, b = msgs[lanes[j - 1]], msgs[lanes[j]]
            if not (a[0] == b[0] and a[3] == b[3] and a[3] != 0 and a[1] + a[3] == b[1] and a[2] + a[3] == b[2]):
                break
            j += 1
        runs[lanes[i]] = j - i
        i = j
    return runs


def test_full_warp_of_contiguous_pieces_becomes_one_message():
    msgs = [(3, 0x1000 + 64 * l, 0x9000 + 64 * l, 64) for l in range(32)]
    assert _plan(0xFFFFFFFF, msgs) == [32] + [0] * 31


def test_runs_break_on_pe_size_gap_and_inactive_lanes_are_skipped():
    msgs = [(1, 0x1000 + 8 * l, 0x5000 + 8 * l, 8) for l in range(32)]
    msgs[8] = (2, msgs[8][1], msgs[8][2], 8)              # other PE: lanes 8 and 9 start new runs
    msgs[20] = (1, msgs[20][1] + 8, msgs[20][2] + 8, 8)   # gap in front of lane 20 (and behind it)
    got = _plan(0xFFFFFFFF, msgs)
    assert got == _brute(0xFFFFFFFF, msgs)
    assert got[0] == 8 and got[8] == 1 and got[9] == 11 and got[20] == 1 and got[21] == 11
    # lanes 4..7 inactive: lane 8's predecessor is lane 3, whose piece does not touch it
    active = 0xFFFFFFFF & ~0xF0
    msgs = [(1, 0x1000 + 8 * l, 0x5000 + 8 * l, 8) for l in range(32)]
    got = _plan(active, msgs)
    assert got[0] == 4 and got[8] == 24 and all(got[l] == 0 for l in (4, 5, 6, 7))
    # compacted addresses over the active lanes only: one run again
    lanes = [l for l in range(32) if active >> l & 1]
    msgs = [(1, 0, 0, 0)] * 32
    for i, l in enumerate(lanes):
        msgs[l] = (1, 0x1000 + 8 * i, 0x5000 + 8 * i, 8)
    assert _plan(active, msgs)[0] == 28


def test_lane_plan_matches_a_lane_by_lane_walk_on_random_warps():
    rng = random.Random(7)
    for _ in range(300):
        active = rng.getrandbits(32) | (1 << rng.randrange(32))
        msgs, dst, src = [], 0x10000, 0x80000
        for l in range(32):
            size = rng.choice([8, 8, 8, 16])
            if rng.random() < 0.2:
                dst += rng.choice([8, 64])
            pe = 1 if rng.random() < 0.9 else 2
            msgs.append((pe, dst, src, size))
            if active >> l & 1:
                dst += size
                src += size
        got = _plan(active, msgs)
        assert got == _brute(active, msgs)
        # every active lane is covered by exactly one leader
        assert sum(got) == bin(active).count("1")


def test_list_form_merges_runs_in_place():
    m = [(1, 100, 500, 10), (1, 110, 510, 10), (1, 120, 520, 10), (2, 130, 530, 10), (2, 140, 540, 10),
         (2, 160, 560, 10), (2, 170, 570, 20)]
    assert rt._C().coalesce_merge_runs(m) == [(1, 100, 500, 30), (2, 130, 530, 20), (2, 160, 560, 10), (2, 170, 570, 20)]
    assert rt._C().coalesce_merge_runs([]) == []


def test_ring_consumer_executes_a_run_of_puts_as_one_transfer(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=2, heap_size="4M", backend="host")
    C = shm.runtime._C()
    p = C.proxy_start()
    try:
        src = shm.zeros(256, torch.int64)
        dst = shm.zeros(256, torch.int64)
        src.copy_(torch.arange(256) + 1000)
        PUT, GET, FADD = 1, 2, 3
        ctr = shm.zeros(1, torch.int64)
        C.proxy_set_coalesce(p, True)
        # While the consumer sleeps on the first command the others are published behind it.
        C.proxy_inject_delay_ms(p, 300)
        for i in range(16):
            assert C.proxy_submit(p, PUT, 1, dst.data_ptr() + 64 * i, src.data_ptr() + 64 * i, 64, 0, 0, 1, False, 5000)[0] == 0
        # a piece that does not follow on, then one to another PE
        assert C.proxy_submit(p, PUT, 1, dst.data_ptr() + 64 * 20, src.data_ptr() + 64 * 20, 64, 0, 0, 1, False, 5000)[0] == 0
        assert C.proxy_submit(p, PUT, 0, dst.data_ptr() + 64 * 21, src.data_ptr() + 64 * 21, 64, 0, 0, 1, False, 5000)[0] == 0
        C.proxy_inject_delay_ms(p, 0)
        rc, _ = C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 1, 0, 0, 8, True, 10000)
        assert rc == 0
        got = shm.local_view(dst, 1)
        assert torch.equal(got[:128], torch.arange(128) + 1000)
        assert torch.equal(got[160:168], torch.arange(160, 168) + 1000) and int(got[130]) == 0
        assert torch.equal(shm.local_view(dst, 0)[168:176], torch.arange(168, 176) + 1000)
        # all fifteen followers on an idle machine; under load the consumer may wake up before the last ones are in
        assert 8 <= C.proxy_merged(p) <= 15
        # blocking producers inside a run are acknowledged one by one: gets issued from two threads
        import threading
        back = shm.zeros(256, torch.int64)
        C.proxy_inject_delay_ms(p, 100)
        assert C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 1, 0, 0, 8, False, 5000)[0] == 0
        C.proxy_inject_delay_ms(p, 0)
        rcs = [None, None]

        def getter(k):
            rcs[k] = C.proxy_submit(p, GET, 1, back.data_ptr() + 512 * k, dst.data_ptr() + 512 * k, 512, 0, 0, 1, True, 10000)[0]
        ts = [threading.Thread(target=getter, args=(k,)) for k in range(2)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        assert rcs == [0, 0]
        assert torch.equal(shm.local_view(back, 0)[:128], torch.arange(128) + 1000)
        # the debug dump of a slot names its state and operation; blocking commands leave their completion behind
        text = C.proxy_describe_command(p, 0)
        assert text.startswith("slot 0 of ") and ("op put" in text or "op get" in text or "op amo_fadd" in text), text
        assert "completion 0 of" in C.proxy_describe_completion(p, 0)
        # with merging off nothing is merged
        C.proxy_set_coalesce(p, False)
        before = C.proxy_merged(p)
        C.proxy_inject_delay_ms(p, 100)
        for i in range(4):
            assert C.proxy_submit(p, PUT, 1, dst.data_ptr() + 64 * i, src.data_ptr() + 64 * i, 64, 0, 0, 1, False, 5000)[0] == 0
        C.proxy_inject_delay_ms(p, 0)
        assert C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 0, 0, 0, 8, True, 10000)[0] == 0
        assert C.proxy_merged(p) == before
    finally:
        C.proxy_stop(p)
        shm.finalize()
