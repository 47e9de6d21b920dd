"""Builds the example programs and runs them: alone on one GPU, and as two processes when two GPUs are
visible. Every example prints PASS / FAIL per PE and exits non-zero on failure, like the reference's."""
import os
import shutil
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples")
PROGS = ["getmem", "put_signal", "broadcast", "alltoall", "allreduce", "team_reduce"]


@pytest.fixture(scope="module")
def built():
    missing = [p for p in PROGS if not os.path.exists(os.path.join(EX, "build", p))]
    if missing:
        if shutil.which("nvcc") is None:
            pytest.skip("examples are not built and nvcc is not available")
        out = subprocess.run(["make", "-C", EX], capture_output=True, text=True, timeout=1200)
        assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    return os.path.join(EX, "build")


def run(cmd, world, tmp_path):
    env = dict(os.environ, ROCSHMEM_BOOTSTRAP_DIR=str(tmp_path), ROCSHMEM_HEAP_SIZE="512M", NCCL_NVLS_ENABLE="0")
    if world > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", "29631"] + cmd
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.count("PASS") == world and "FAIL" not in out.stdout, out.stdout[-2000:]


@pytest.mark.parametrize("prog", PROGS)
def test_cuda_example_single_pe(built, prog, tmp_path):
    run([os.path.join(built, prog)], 1, tmp_path)


@pytest.mark.parametrize("prog", PROGS)
def test_cuda_example_two_pes(built, prog, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run(["--no-python", os.path.join(built, prog)], 2, tmp_path)


@pytest.mark.parametrize("script", ["allreduce.py", "moe_layer.py", "tp_mlp.py"])
def test_python_example(script, tmp_path):
    world = 2 if torch.cuda.device_count() >= 2 else 1
    cmd = [os.path.join(EX, "python", script)]
    run(cmd if world > 1 else [sys.executable] + cmd, world, tmp_path)


@pytest.mark.parametrize("test", ["put", "get", "amo_fadd", "pingpong", "barrier", "allreduce", "broadcast", "alltoall",
                                  # per-scope forms, selected as the reference does, by number or by name
                                  "31", "ctx_get_thread", "amo_swap", "put_signal_wg", "pingall"])
def test_functional_driver(test, tmp_path):
    """The command-line performance driver prints one table row per message size (two PEs on one GPU)."""
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "functional_driver.py"), "-a", test, "-s", "65536", "-m", "4096",
           "--local-pes", "2", "--loop", "3", "--skip", "1", "-z", "128"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, ROCSHMEM_BOOTSTRAP_DIR=str(tmp_path)))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    rows = [l for l in out.stdout.splitlines() if l.strip() and l.strip()[0].isdigit()]
    assert len(rows) >= 1, out.stdout
    assert all(len(r.split()) == 5 for r in rows), out.stdout
