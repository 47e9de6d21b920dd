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
                                      "gpu_proxied_collectives", "gpu_moe", "gpu_tp_fused", "gpu_models"])
def test_scenario(scenario, world):
    if world == 0:
        pytest.skip("needs at least two GPUs")
    results = run_ranks(scenario, world, timeout=300, env_extra=CUDA_ENV)
    assert_all_ok(results)
    if scenario in ("gpu_device_suite", "gpu_library_collectives"):
        print(results[0][1][-400:])
