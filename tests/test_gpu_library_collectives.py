"""The library's stream-ordered collective kernels (allreduce, broadcast, fcollect, alltoall, barrier) with four
PEs on one GPU, on the world team and on sub-teams, against fp64 host references; and a team slot that is reused
by a team with other members after its first occupant ran a different number of library kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NPES = 4


@pytest.fixture(scope="module")
def shm():
    import rocshmem_b200 as s
    if s.is_initialized():
        s.finalize()
    s.init(n_local=NPES, heap_size="256M", ROCSHMEM_WAIT_TIMEOUT_MS=5000)
    yield s
    torch.cuda.synchronize()
    s.finalize()


def clean(shm):
    torch.cuda.synchronize()
    for l in range(NPES):
        err = shm.get_error(l)
        assert err["count"] == 0, err


def fill(shm, t, fn):
    for l in range(NPES):
        shm.local_view(t, l).copy_(fn(l).to(t.dtype).to(shm.device()))
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [256, 5000, 1 << 20])
@pytest.mark.parametrize("members", [(0, 1, 4), (0, 2, 2), (1, 1, 3)])
def test_allreduce_on_teams_against_fp64(shm, dtype, n, members):
    from rocshmem_b200.ops import collectives as coll
    start, stride, size = members
    pes = [start + i * stride for i in range(size)]
    team = shm.team_world() if members == (0, 1, NPES) else shm.team_world().split_strided(start, stride, size)
    src, dst = shm.zeros(n, dtype), shm.zeros(n, dtype)
    host = [torch.randn(n, generator=torch.Generator().manual_seed(7 * l + n)).to(dtype) for l in range(NPES)]
    fill(shm, src, lambda l: host[l])
    for algo in (shm.ALLREDUCE_AUTO, shm.ALLREDUCE_ONE_SHOT, shm.ALLREDUCE_TWO_SHOT):
        fill(shm, dst, lambda l: torch.full((n,), -7.0))
        coll.allreduce_async(dst, src, team=team, algo=algo)
        clean(shm)
        want = sum(host[p].double() for p in pes)
        tol = 1e-5 if dtype == torch.float32 else 3e-2
        for l in range(NPES):
            got = shm.local_view(dst, l).double().cpu()
            if l in pes:
                assert (got - want).abs().max().item() <= tol * max(1.0, want.abs().max().item()), (algo, l)
            else:
                assert torch.all(got == -7.0), "a PE outside the team was written"
    if team.handle != shm.team_world().handle:
        team.destroy()
    shm.free(dst)
    shm.free(src)


@pytest.mark.parametrize("nbytes", [4096, 1 << 20, (3 << 20) + 4096])
def test_broadcast_fcollect_alltoall(shm, nbytes):
    from rocshmem_b200.ops import collectives as coll
    src = shm.zeros(nbytes * NPES, torch.uint8)
    dst = shm.zeros(nbytes * NPES, torch.uint8)
    host = [torch.randint(0, 256, (nbytes * NPES,), generator=torch.Generator().manual_seed(31 * l + 1),
                          dtype=torch.uint8) for l in range(NPES)]
    fill(shm, src, lambda l: host[l])
    coll.fcollect_async(dst, src[:nbytes])
    clean(shm)
    for l in range(NPES):
        got = shm.local_view(dst, l).cpu().view(NPES, nbytes)
        assert all(torch.equal(got[p], host[p][:nbytes]) for p in range(NPES))
    coll.alltoall_async(dst, src)
    clean(shm)
    for l in range(NPES):
        got = shm.local_view(dst, l).cpu().view(NPES, nbytes)
        assert all(torch.equal(got[p], host[p].view(NPES, nbytes)[l]) for p in range(NPES))
    root = 2
    fill(shm, dst, lambda l: torch.zeros(nbytes * NPES))
    coll.broadcast_async(dst[:nbytes], src[:nbytes], root)
    clean(shm)
    for l in range(NPES):
        got = shm.local_view(dst, l).cpu()[:nbytes]
        if l == root:
            assert torch.all(got == 0), "the root's dest stays untouched"
        else:
            assert torch.equal(got, host[root][:nbytes])
    shm.free(dst)
    shm.free(src)


def test_a_reused_team_slot_starts_from_clean_library_epochs(shm):
    """Team {0, 2} runs three library kernels and is destroyed; {0, 1} then lands in the same slot. PE 0 has run
    three kernels in that slot, PE 1 none: without cleared epochs and flags PE 0 would wait for a flag value that
    PE 1 never writes (the wait is bounded, so the failing form times out rather than hangs)."""
    from rocshmem_b200.ops import collectives as coll
    n = 4096
    src, dst = shm.zeros(n, torch.float32), shm.zeros(n * NPES, torch.float32)
    fill(shm, src, lambda l: torch.full((n,), float(l + 1)))
    first = shm.team_world().split_strided(0, 2, 2)
    for _ in range(3):
        coll.allreduce_async(dst[:n], src, team=first)
    clean(shm)
    assert shm.local_view(dst, 0)[0].item() == 1.0 + 3.0
    slot_handle = first.handle
    first.destroy()
    second = shm.team_world().split_strided(0, 1, 2)
    assert second.handle == slot_handle, "the test expects the freed slot to be taken again"
    coll.allreduce_async(dst[:n], src, team=second)
    clean(shm)
    assert shm.local_view(dst, 0)[0].item() == 1.0 + 2.0 and shm.local_view(dst, 1)[n - 1].item() == 3.0
    coll.fcollect_async(dst[:2 * n], src, team=second)
    clean(shm)
    got = shm.local_view(dst, 1).cpu()[:2 * n].view(2, n)
    assert torch.all(got[0] == 1.0) and torch.all(got[1] == 2.0)
    second.destroy()
    shm.free(dst)
    shm.free(src)
