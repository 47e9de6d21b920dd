"""Multi-process scenarios on the host-memory backend: real processes, real descriptor passing,
the same runtime code as on GPUs."""
import pytest

from mp_util import assert_all_ok, run_ranks


@pytest.mark.parametrize("world", [2, 4])
def test_host_api_plumbing(world):
    assert_all_ok(run_ranks("host_plumbing", world))


def test_torch_store_bootstrap():
    assert_all_ok(run_ranks("store_bootstrap", 3))


def test_teams_split_translate_capacity():
    assert_all_ok(run_ranks("teams", 4))


@pytest.mark.parametrize("fail,expect", [
    (None, "world,lower,upper,even,rest"),
    # the world object fails on one rank: nobody has a mapping, and no team tries for one
    ((2, "bind:0"), ""),
    # rank 2's third object is the even team {0, 2}: both of its members go without, the other teams are untouched
    ((2, "add:2"), "world,lower,upper,rest"),
    # rank 0 creates the lower team's object (its second); rank 3 imports the upper team's
    ((0, "create:1"), "world,upper,even,rest"),
    ((3, "import:1"), "world,lower,even,rest"),
])
def test_multicast_objects_of_world_and_split_teams_are_all_or_nothing(fail, expect):
    """The host provider's stand-in for the NVLink multicast object: creation on the first member, descriptor to the
    others, agreement after every step, tear-down at destroy and finalize, as four real processes."""
    env = {"ROCSHMEM_HOST_FAKE_MULTICAST": "1", "EXPECT_MULTICAST": expect}
    if fail is not None:
        env.update(FAKE_MC_FAIL_RANK=fail[0], FAKE_MC_FAIL_SPEC=fail[1])
    assert_all_ok(run_ranks("team_multicast_standin", 4, env_extra=env))


@pytest.mark.parametrize("world", [2, 3])
def test_host_collectives(world):
    assert_all_ok(run_ranks("collectives_host", world))


def test_wait_family_between_processes():
    assert_all_ok(run_ranks("wait_and_signal", 3))


@pytest.mark.parametrize("world", [2, 3])
def test_proxy_ring_runs_host_collectives(world):
    """Reverse-offload command set beyond RMA: fence, P, broadcast, reduce, fcollect, alltoall."""
    assert_all_ok(run_ranks("proxy_collectives", world))


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_dispatch_combine_through_the_host_api(world):
    assert_all_ok(run_ranks("ep_host", world))


def test_moe_layer_over_the_host_api():
    assert_all_ok(run_ranks("moe_layer_host", 3))


def test_process_grid_teams_and_pipeline_channel():
    assert_all_ok(run_ranks("parallel_layout", 4))


def test_back_to_back_collectives_team_reuse_and_many_contexts():
    assert_all_ok(run_ranks("stress_host", 3, timeout=240))


@pytest.mark.parametrize("world", [4, 6, 8])
def test_bruck_and_clustered_schedules_match_the_linear_ones(world):
    assert_all_ok(run_ranks("host_algorithms", world, timeout=240))


def test_threads_per_process_all_to_all_wait_chain_and_large_transfers():
    assert_all_ok(run_ranks("threads_host", 3, timeout=240))


def test_collective_baseline_wrappers_over_gloo():
    assert_all_ok(run_ranks("collective_baselines", 3))


def test_all_to_all_baseline_of_dispatch_and_combine():
    assert_all_ok(run_ranks("ep_collective_baseline", 3, timeout=240))


def test_data_parallel_gradient_buckets():
    assert_all_ok(run_ranks("data_parallel", 3, timeout=240))


def test_sequence_parallel_attention_through_all_to_all_resharding():
    assert_all_ok(run_ranks("ulysses", 4, timeout=240))


def test_ring_exchange_and_ring_attention():
    assert_all_ok(run_ranks("ring_attention", 4, timeout=240))


def test_pipeline_stages_match_the_whole_model():
    assert_all_ok(run_ranks("pipeline_stages", 3, timeout=240))


def test_variable_count_all_to_all():
    assert_all_ok(run_ranks("alltoallv_host", 4, timeout=240))


@pytest.mark.parametrize("world", [3, 4])
def test_reduce_scatter_over_the_host_api(world):
    assert_all_ok(run_ranks("reduce_scatter_host", world, timeout=240))
