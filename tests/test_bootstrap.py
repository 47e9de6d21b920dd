"""Bootstrap channel: file rendezvous, allgather, descriptor passing between processes."""
import multiprocessing as mp
import os
import tempfile

from rocshmem_b200 import _native


def _allgather_worker(d, rank, size, q):
    C = _native.load()
    out = C.file_bootstrap_allgather(d, rank, size, bytes([rank]) * 5, 20000)
    q.put((rank, out))


def test_file_allgather_four_processes():
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as d:
        q = ctx.Queue()
        procs = [ctx.Process(target=_allgather_worker, args=(d, r, 4, q)) for r in range(4)]
        [p.start() for p in procs]
        got = dict(q.get(timeout=60) for _ in range(4))
        [p.join(30) for p in procs]
    want = b"".join(bytes([r]) * 5 for r in range(4))
    assert all(got[r] == want for r in range(4))


def _fd_worker(d, rank, size, q):
    C = _native.load()
    fd = os.memfd_create(f"t{rank}")
    os.write(fd, f"payload-from-{rank}".encode())
    fds = C.exchange_fds_file(d, rank, size, fd, 20000)
    seen = []
    for r, f in enumerate(fds):
        # pread: descriptors passed between processes share one file offset, so lseek + read would race
        seen.append(os.pread(f, 64, 0).decode())
        os.close(f)
    q.put((rank, seen))


def test_descriptor_exchange_three_processes():
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as d:
        q = ctx.Queue()
        procs = [ctx.Process(target=_fd_worker, args=(d, r, 3, q)) for r in range(3)]
        [p.start() for p in procs]
        got = dict(q.get(timeout=60) for _ in range(3))
        [p.join(30) for p in procs]
    for r in range(3):
        assert got[r] == [f"payload-from-{i}" for i in range(3)]


def _fd_group_worker(d, rank, size, members, q):
    C = _native.load()
    fd = -1
    if rank == members[0]:
        fd = os.memfd_create("group")
        os.write(fd, b"from-the-first-member")
    got = C.broadcast_fd_group_file(d, rank, size, members, fd, 20000)
    q.put((rank, os.pread(got, 64, 0).decode()))
    os.close(got)


def test_descriptor_from_the_first_member_of_a_subgroup():
    """Four processes, three of them form a group (not in rank order of the job): the first member's descriptor
    reaches the two others; the process outside the group takes no part."""
    ctx = mp.get_context("spawn")
    members = [2, 0, 3]
    with tempfile.TemporaryDirectory() as d:
        q = ctx.Queue()
        procs = [ctx.Process(target=_fd_group_worker, args=(d, r, 4, members, q)) for r in members]
        [p.start() for p in procs]
        got = dict(q.get(timeout=60) for _ in members)
        [p.join(30) for p in procs]
    assert got == {r: "from-the-first-member" for r in members}


def test_descriptor_group_with_an_absent_sender_times_out():
    C = _native.load()
    import time
    with tempfile.TemporaryDirectory() as d:
        t0 = time.time()
        try:
            C.broadcast_fd_group_file(d, 1, 2, [0, 1], -1, 300)      # rank 0, the sender, never shows up
            raise AssertionError("returned although the sender never joined")
        except RuntimeError as e:
            assert "timed out" in str(e)
        assert time.time() - t0 < 10


def test_missing_rank_times_out_instead_of_hanging():
    C = _native.load()
    import time
    with tempfile.TemporaryDirectory() as d:
        t0 = time.time()
        try:
            C.file_bootstrap_allgather(d, 0, 2, b"x", 300)
            raise AssertionError("allgather returned although rank 1 never joined")
        except RuntimeError as e:
            assert "timed out" in str(e)
        assert time.time() - t0 < 10
