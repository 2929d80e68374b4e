"""NUMA helpers against a fake sysfs tree."""
import os

from dlslime_b200.utils import numa


def test_cpulist_and_pci_node(tmp_path):
    root = tmp_path
    (root / "devices/system/node/node1").mkdir(parents=True)
    (root / "devices/system/node/node1/cpulist").write_text("4-7,12,14-15\n")
    (root / "bus/pci/devices/0000:3b:00.0").mkdir(parents=True)
    (root / "bus/pci/devices/0000:3b:00.0/numa_node").write_text("1\n")
    assert numa.node_cpus(1, str(root)) == {4, 5, 6, 7, 12, 14, 15}
    assert numa.node_cpus(3, str(root)) == set()
    assert numa.pci_numa_node("0000:3B:00.0", str(root)) == 1
    assert numa.pci_numa_node("0000:ff:00.0", str(root)) == -1
    assert numa.bind_to_numa_node(-1, str(root)) is False
    assert numa.bind_to_numa_node(3, str(root)) is False


def test_bind_to_existing_cpus(tmp_path):
    allowed = sorted(os.sched_getaffinity(0))
    root = tmp_path
    (root / "devices/system/node/node0").mkdir(parents=True)
    (root / "devices/system/node/node0/cpulist").write_text(str(allowed[0]) + "\n")
    try:
        assert numa.bind_to_numa_node(0, str(root)) is True
        assert os.sched_getaffinity(0) == {allowed[0]}
    finally:
        os.sched_setaffinity(0, allowed)
