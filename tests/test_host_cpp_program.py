"""Builds the host-only C++ programs tests/cpp/host_api_sos.cpp, host_threads_sos.cpp and host_patterns_sos.cpp with g++ against the
runtime library and runs them as several processes on the CPU shared-memory backend: the typed C++ host API (put /
get / p / g, atomics, waits, collectives, teams, contexts, rocshmem_ptr; then several threads per process, each
with its own context) end to end, as the reference's SOS programs do for its host API."""
import os
import shutil
import subprocess

import pytest

from rocshmem_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "rocshmem_b200", "csrc", "include")
LIB = os.path.join(ROOT, "rocshmem_b200", "lib")


@pytest.fixture(scope="module")
def programs(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("needs g++")
    if not _build.is_built():
        _build.build(with_tests=False)
    out = {}
    for name in ("host_api_sos", "host_threads_sos", "host_patterns_sos"):
        exe = str(tmp_path_factory.mktemp("sos") / name)
        cmd = ["g++", "-std=c++17", "-O1", "-g", f"-I{INC}", os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", exe,
               f"-L{LIB}", "-lrocshmem_b200", f"-Wl,-rpath,{LIB}", "-lpthread"]
        build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert build.returncode == 0, build.stderr[-3000:]
        out[name] = exe
    return out


@pytest.mark.parametrize("name,world", [("host_api_sos", 2), ("host_api_sos", 5), ("host_threads_sos", 3),
                                        ("host_patterns_sos", 2), ("host_patterns_sos", 5)])
def test_cpp_host_programs_on_the_cpu_backend(programs, name, world, tmp_path):
    program = programs[name]
    kv = tmp_path / "kv"
    kv.mkdir()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), ROCSHMEM_BACKEND="host",
                   ROCSHMEM_HEAP_SIZE="64M", ROCSHMEM_BOOTSTRAP_DIR=str(kv), ROCSHMEM_WAIT_TIMEOUT_MS="30000")
        procs.append(subprocess.Popen([program], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=180)
            outs.append((p.returncode, out))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (rc, out) in enumerate(outs):
        assert rc == 0 and f"[pe {r}] PASS" in out, (r, rc, out[-2000:])


def test_launcher_runs_ranks_tags_output_and_propagates_failures(programs):
    """python -m rocshmem_b200.launch: the mpirun of this runtime."""
    import io
    import sys
    import time

    from rocshmem_b200 import launch
    out = io.StringIO()
    rc = launch.launch([programs["host_api_sos"]], 3, backend="host", timeout_s=120, out=out,
                       extra_env={"ROCSHMEM_HEAP_SIZE": "16M"})
    text = out.getvalue()
    assert rc == 0, text[-2000:]
    assert all(f"[{r}] [pe {r}] PASS" in text for r in range(3))
    # one rank fails: its exit code comes back and the ranks that would run on are terminated
    script = "import os, sys, time\nif os.environ['RANK'] == '1': sys.exit(7)\ntime.sleep(60)"
    t0 = time.time()
    rc = launch.launch([sys.executable, "-c", script], 3, timeout_s=50, out=io.StringIO())
    assert rc == 7 and time.time() - t0 < 30
    # time-out
    rc = launch.launch([sys.executable, "-c", "import time; time.sleep(60)"], 2, timeout_s=1.0, out=io.StringIO())
    assert rc == 124
    # command line form
    assert launch.main(["-n", "2", "--no-tag", "--", sys.executable, "-c", "import os; assert os.environ['WORLD_SIZE'] == '2'"]) == 0


def test_global_exit_ends_every_rank_with_the_status(programs):
    """One PE calls rocshmem_global_exit(7) while the others wait on a word nobody writes (the reference's
    global_exit program): the job ends with that status instead of waiting for the time-out."""
    import io
    import time

    from rocshmem_b200 import launch
    t0 = time.time()
    rc = launch.launch([programs["host_patterns_sos"], "exit"], 3, backend="host", timeout_s=100, out=io.StringIO(),
                       extra_env={"ROCSHMEM_HEAP_SIZE": "16M", "ROCSHMEM_WAIT_TIMEOUT_MS": "60000"})
    assert rc == 7 and time.time() - t0 < 40


def test_repeated_launches_on_one_port_do_not_see_each_others_rendezvous_files(programs):
    """Without ROCSHMEM_BOOTSTRAP_DIR the rendezvous directory is derived from the port, the run id and the
    launching process, so a second job on the same port starts clean, and directories whose launcher is gone are
    removed by the next job."""
    import glob
    import sys
    env = {k: v for k, v in os.environ.items() if k != "ROCSHMEM_BOOTSTRAP_DIR"}
    env.update(ROCSHMEM_BACKEND="host", ROCSHMEM_HEAP_SIZE="16M")
    pattern = f"/dev/shm/rocshmem_b200.{os.getuid()}.29677.*"
    for attempt in range(2):
        out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--no-python", "--nnodes=1",
                              "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29677",
                              programs["host_api_sos"]], env=env, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0 and out.stdout.count("PASS") == 2, (attempt, out.stdout[-2000:] + out.stderr[-3000:])
        assert len(glob.glob(pattern)) == 1          # the first job's directory was purged by the second
    for d in glob.glob(pattern):
        shutil.rmtree(d, ignore_errors=True)
