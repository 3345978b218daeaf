"""Host affinity helper against a fake sysfs tree (nothing of the real machine is changed)."""
from configurable_hierarchical_allreduce_algorithms_b200.utils import affinity


def _fake(tmp_path, nodes):
    for n, cpus in nodes.items():
        d = tmp_path / "devices" / "system" / "node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpus + "\n")
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    return dev


def test_cpulist_grammar():
    assert affinity.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert affinity.parse_cpulist("") == []


def test_gpu_on_second_node_is_found(tmp_path):
    dev = _fake(tmp_path, {0: "0-15", 1: "16-31"})
    (dev / "numa_node").write_text("1\n")
    node, cpus = affinity.numa_of_pci("0000:1b:00.0", str(tmp_path))
    assert node == 1 and cpus == list(range(16, 32))
    rec = affinity.bind_to_gpu(0, str(tmp_path), apply=False, pci_addr="0000:1b:00.0")
    assert rec["numa_node"] == 1 and rec["cpus"] == 16 and rec["nodes"] == 2 and not rec["bound"]


def test_single_node_machine_is_left_alone(tmp_path):
    dev = _fake(tmp_path, {0: "0-31"})
    (dev / "numa_node").write_text("0\n")
    rec = affinity.bind_to_gpu(0, str(tmp_path), apply=True, pci_addr="0000:1b:00.0")
    assert not rec["bound"] and "why_not" in rec
    (dev / "numa_node").write_text("-1\n")
    assert affinity.bind_to_gpu(0, str(tmp_path), apply=True, pci_addr="0000:1b:00.0")["numa_node"] == -1
