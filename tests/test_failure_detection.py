"""Failure detection without touching a GPU: the failure is made on the host (a rank that never
joins, a rank that leaves between steps, a dropped proxy command) and must surface as an error or
status, never as a hang."""
import time

import torch

from mp_util import assert_all_ok, run_ranks


def test_rank_that_never_joins_is_reported():
    t0 = time.time()
    results = run_ranks("late_rank", 2, timeout=90, args=(4,))
    assert_all_ok(results)
    assert "detected" in results[0][1]
    assert time.time() - t0 < 80


def test_rank_leaves_between_steps_and_survivors_continue():
    assert_all_ok(run_ranks("rank_leaves", 3, timeout=120))


def test_team_destroy_returns_when_a_member_of_a_multicast_team_has_left():
    """team_destroy of a team with a multicast object is collective; a member that left must cost the survivor the
    rendezvous time-out and nothing more (host provider's stand-in for the object, three CPU processes)."""
    t0 = time.time()
    results = run_ranks("team_member_leaves", 3, timeout=120,
                        env_extra={"ROCSHMEM_HOST_FAKE_MULTICAST": 1, "ROCSHMEM_TEST_TIMEOUT": 4})
    assert_all_ok(results)
    assert "team_destroy" in results[0][1]          # the survivor says what it gave up waiting for
    assert time.time() - t0 < 90


def test_proxy_ring_executes_and_reports_dropped_commands(fresh_runtime):
    shm = fresh_runtime
    shm.init(n_local=2, heap_size="4M", backend="host")
    C = shm.runtime._C()
    p = C.proxy_start()
    try:
        src = shm.zeros(64, torch.int64)
        dst = shm.zeros(64, torch.int64)
        src.copy_(torch.arange(64))
        PUT, GET, FADD, CAS = 1, 2, 3, 4
        rc, _ = C.proxy_submit(p, PUT, 1, dst.data_ptr(), src.data_ptr(), 64 * 8, 0, 0, 1, True, 2000)
        assert rc == 0 and torch.equal(shm.local_view(dst, 1), torch.arange(64))
        ctr = shm.zeros(1, torch.int64)
        olds = [C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 3, 0, 0, 8, True, 2000)[1] for _ in range(5)]
        assert olds == [0, 3, 6, 9, 12]
        rc, old = C.proxy_submit(p, CAS, 1, ctr.data_ptr(), 0, 100, 15, 0, 8, True, 2000)
        assert rc == 0 and old == 15 and int(shm.local_view(ctr, 1)[0]) == 100
        # more commands than ring slots, fire-and-forget, then a blocking one to drain
        for i in range(2000):
            assert C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 1, 0, 0, 8, False, 2000)[0] == 0
        rc, old = C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 0, 0, 0, 8, True, 5000)
        assert rc == 0 and old == 2100
        # injected loss: the blocking producer gets an error after its budget, the ring keeps working
        C.proxy_inject_drop(p, 1)
        t0 = time.time()
        rc, _ = C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 1, 0, 0, 8, True, 200)
        assert rc == 1 and 0.15 < time.time() - t0 < 5
        rc, old = C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 1, 0, 0, 8, True, 2000)
        assert rc == 0 and old == 2100
        # injected delay longer than the budget: time-out, then the late completion is harmless
        C.proxy_inject_delay_ms(p, 300)
        rc, _ = C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 1, 0, 0, 8, True, 50)
        assert rc == 1
        C.proxy_inject_delay_ms(p, 0)
        time.sleep(0.5)
        rc, old = C.proxy_submit(p, FADD, 1, ctr.data_ptr(), 0, 0, 0, 0, 8, True, 2000)
        assert rc == 0 and old in (2101, 2102)
        executed, dropped = C.proxy_counts(p)
        assert dropped == 1 and executed >= 2008
    finally:
        C.proxy_stop(p)
        shm.finalize()


def test_world_shrinks_when_a_middle_rank_leaves_and_survivors_restore_their_heap():
    results = run_ranks("elastic_shrink", 4, timeout=180)
    assert_all_ok(results)
    assert "rank 2 left" in results[2][1]


def test_survivors_notice_a_silent_departure_and_rebuild_the_world():
    t0 = time.time()
    results = run_ranks("elastic_unplanned", 3, timeout=150, env_extra={"ROCSHMEM_TEST_TIMEOUT": 6})
    assert_all_ok(results)
    assert time.time() - t0 < 120


def test_world_grows_when_a_process_joins_between_steps():
    assert_all_ok(run_ranks("elastic_grow", 3, timeout=180))
