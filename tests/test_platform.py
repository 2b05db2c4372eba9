"""NUMA helpers against a fake sysfs tree (no GPU, no real binding)."""
import os

from xllm_wxh_b200.platform import numa


def _fake_sysfs(tmp_path):
    root = tmp_path / "sys"
    for n, cpus in ((0, "0-3"), (1, "4-7,12")):
        d = root / "devices/system/node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpus + "\n")
    for bus, node in (("0000:1b:00.0", 0), ("0000:9c:00.0", 1), ("0000:aa:00.0", -1)):
        d = root / "bus/pci/devices" / bus
        d.mkdir(parents=True)
        (d / "numa_node").write_text(f"{node}\n")
    return str(root)


def test_parse_cpulist():
    assert numa.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert numa.parse_cpulist("") == []


def test_sysfs_lookups(tmp_path):
    root = _fake_sysfs(tmp_path)
    assert numa.num_numa_nodes(root) == 2
    assert numa.node_cpus(1, root) == [4, 5, 6, 7, 12]
    assert numa.pci_numa_node("0000:9C:00.0", root) == 1          # case-insensitive bus id
    assert numa.pci_numa_node("0000:aa:00.0", root) == -1
    assert numa.pci_numa_node("0000:ff:00.0", root) == -1          # unknown device
    assert numa.num_numa_nodes(str(tmp_path / "nothing")) == -1


def test_bind_intersects_with_the_allowed_cpus(tmp_path):
    root = _fake_sysfs(tmp_path)
    calls = []
    rc = numa.bind_to_node(1, root, set_memory=False, setaffinity=lambda pid, cpus: calls.append((pid, set(cpus))),
                           getaffinity=lambda pid: {0, 1, 5, 6, 12})
    assert rc == 0 and calls == [(0, {5, 6, 12})]
    # a cpuset without any CPU of the node: left alone
    calls.clear()
    rc = numa.bind_to_node(1, root, set_memory=False, setaffinity=lambda pid, cpus: calls.append(cpus),
                           getaffinity=lambda pid: {0, 1})
    assert rc == -2 and calls == []
    assert numa.bind_to_node(-1, root) == -1


def test_refused_affinity_is_reported_not_raised(tmp_path):
    root = _fake_sysfs(tmp_path)

    def refuse(pid, cpus):
        raise OSError("operation not permitted")
    assert numa.bind_to_node(0, root, set_memory=False, setaffinity=refuse, getaffinity=lambda pid: set(range(16))) == -3
