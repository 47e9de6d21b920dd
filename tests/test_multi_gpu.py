"""One PE per process and per GPU. Skipped unless at least two GPUs are visible."""
import pytest
import torch

from mp_util import assert_all_ok, run_ranks

pytestmark = pytest.mark.gpu


def gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def world_sizes():
    # Two ranks and the largest power of two the box offers (the scenarios at 8 ranks take minutes each).
    n = gpus()
    sizes = [w for w in (2, 4, 8) if w <= n]
    return sorted({sizes[0], sizes[-1]}) if sizes else [0]


CUDA_ENV = {"ROCSHMEM_TEST_BACKEND": "cuda", "NCCL_NVLS_ENABLE": "0"}


@pytest.mark.parametrize("world", world_sizes())
@pytest.mark.parametrize("scenario", ["host_plumbing", "store_bootstrap", "teams", "collectives_host",
                                      "wait_and_signal", "gpu_device_suite", "gpu_library_collectives",
                                      "gpu_team_nvls",
                                      "gpu_proxied_collectives", "gpu_moe", "gpu_tp_fused", "gpu_models",
                                      # the parallelism helpers on their GPU paths (stream-ordered kernels)
                                      "data_parallel", "ulysses", "ring_attention", "pipeline_stages"])
def test_scenario(scenario, world):
    if world == 0:
        pytest.skip("needs at least two GPUs")
    env = dict(CUDA_ENV)
    if scenario == "gpu_proxied_collectives":
        # the waiting kernel and the proxy's kernels need hardware queues of their own (the runtime asks for the same
        # when it is the first to touch CUDA in the process)
        env["CUDA_DEVICE_MAX_CONNECTIONS"] = "32"
    results = run_ranks(scenario, world, timeout=300, env_extra=env)
    assert_all_ok(results)
    if scenario in ("gpu_device_suite", "gpu_library_collectives"):
        print(results[0][1][-400:])


@pytest.mark.parametrize("name", ["host_api_sos", "host_threads_sos", "host_patterns_sos"])
def test_cpp_host_programs_on_the_cuda_backend(name, tmp_path):
    """The typed C++ host API (and several host threads per process, each with its own context) over real peer
    mappings: the programs of test_host_cpp_program.py, one process per GPU."""
    import os
    import shutil
    import subprocess

    from rocshmem_b200 import _build
    if gpus() < 2:
        pytest.skip("needs at least two GPUs")
    if shutil.which("g++") is None:
        pytest.skip("needs g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    inc = os.path.join(root, "rocshmem_b200", "csrc", "include")
    lib = os.path.join(root, "rocshmem_b200", "lib")
    if not _build.is_built():
        _build.build(with_tests=False)
    exe = str(tmp_path / name)
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", f"-I{inc}", os.path.join(root, "tests", "cpp", name + ".cpp"),
                            "-o", exe, f"-L{lib}", "-lrocshmem_b200", f"-Wl,-rpath,{lib}", "-lpthread"],
                           capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-3000:]
    world = 2
    kv = tmp_path / "kv"
    kv.mkdir()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), ROCSHMEM_BACKEND="cuda",
                   ROCSHMEM_HEAP_SIZE="64M", ROCSHMEM_BOOTSTRAP_DIR=str(kv), ROCSHMEM_WAIT_TIMEOUT_MS="10000",
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([exe], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=90)
            outs.append((p.returncode, out))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (rc, out) in enumerate(outs):
        assert rc == 0 and f"[pe {r}] PASS" in out, (r, rc, out[-2000:])

