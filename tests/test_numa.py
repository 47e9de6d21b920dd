"""NUMA placement helper against a fake sysfs tree (no GPU, no NUMA machine needed)."""
import os

from rocshmem_b200.utils import numa


def test_cpulist_parsing_and_node_lookup(tmp_path):
    node = tmp_path / "devices/system/node"
    (node / "node1").mkdir(parents=True)
    (node / "node1" / "cpulist").write_text("48-95,144-191\n")
    (node / "online").write_text("0-1\n")
    cpus = numa.node_cpus(1, str(tmp_path))
    assert len(cpus) == 96 and min(cpus) == 48 and max(cpus) == 191 and 100 not in cpus
    assert numa.online_nodes(str(tmp_path)) == [0, 1]
    assert numa.node_cpus(7, str(tmp_path)) == set()


def test_binding_without_numa_information_changes_nothing(tmp_path):
    before = os.sched_getaffinity(0)
    info = numa.bind_to_device_node(0, sysfs=str(tmp_path))   # no GPU, empty sysfs
    assert info["node"] is None and info["cpus"] == 0 and "no NUMA node" in info["note"]
    assert os.sched_getaffinity(0) == before
