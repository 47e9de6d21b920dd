"""Helpers to run a scenario as several PE processes on one machine."""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(scenario: str, world: int, *, timeout: float = 120.0, env_extra=None, args=(),
              expect_fail_ranks=()):
    """Start ``world`` processes of ``mp_worker.py <scenario>``; return [(returncode, output)]."""
    port = free_port()
    tmp = tempfile.mkdtemp(prefix="rocshmem_b200_test_")
    procs = []
    for rank in range(world):
        env = dict(os.environ)
        env.update({
            "RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
            "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "ROCSHMEM_TEST_TMP": tmp,
            "PYTHONPATH": ROOT + os.pathsep + env.get("PYTHONPATH", ""),
        })
        if env_extra:
            env.update({k: str(v) for k, v in env_extra.items()})
        procs.append(subprocess.Popen(
            [sys.executable, os.path.join(HERE, "mp_worker.py"), scenario, *map(str, args)],
            env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    results = []
    for rank, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed: timeout]"
        results.append((p.returncode, out))
    return results


def assert_all_ok(results):
    for rank, (rc, out) in enumerate(results):
        assert rc == 0, f"rank {rank} failed (rc={rc}):\n{out[-4000:]}"
