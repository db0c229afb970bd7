"""CPU-affinity helper that places a rank's pinned input buffers next to its GPU."""

import os

from pcie_ep_b200.utils.numa import bind_to_device_numa_node, node_cpus, parse_cpu_list


def test_parse_cpu_list_formats():
    assert parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert parse_cpu_list("5") == [5]
    assert parse_cpu_list("") == []


def test_node_cpus_reads_a_fake_sysfs(tmp_path):
    (tmp_path / "node1").mkdir()
    (tmp_path / "node1" / "cpulist").write_text("2-3\n")
    assert node_cpus(1, str(tmp_path)) == [2, 3]
    assert node_cpus(7, str(tmp_path)) == []


def test_bind_restricts_to_the_nodes_cpus_and_ignores_unknown_nodes(tmp_path):
    before = os.sched_getaffinity(0)
    try:
        assert bind_to_device_numa_node(0, numa_node=-1, sysfs_root=str(tmp_path)) is None
        assert bind_to_device_numa_node(0, numa_node=3, sysfs_root=str(tmp_path)) is None  # no such node
        keep = sorted(before)[:1]
        (tmp_path / "node0").mkdir()
        (tmp_path / "node0" / "cpulist").write_text(",".join(str(c) for c in keep) + ",99999\n")
        assert bind_to_device_numa_node(0, numa_node=0, sysfs_root=str(tmp_path)) == 0
        assert os.sched_getaffinity(0) == set(keep)
        assert os.sched_getaffinity(0) <= before
    finally:
        os.sched_setaffinity(0, before)


def test_fastest_upload_node_is_chosen_by_measurement(tmp_path):
    from pcie_ep_b200.utils.numa import available_nodes, bind_to_fastest_upload_node

    before = os.sched_getaffinity(0)
    cpus = sorted(before)
    if len(cpus) < 2:
        return
    for node, cpu in enumerate(cpus[:2]):
        (tmp_path / f"node{node}").mkdir()
        (tmp_path / f"node{node}" / "cpulist").write_text(f"{cpu}\n")
    assert available_nodes(str(tmp_path)) == [0, 1]
    try:
        seen = []

        def fake(device, num_bytes):
            seen.append(sorted(os.sched_getaffinity(0)))
            return 50.0 if seen[-1] == [cpus[1]] else 20.0

        result = bind_to_fastest_upload_node(0, sysfs_root=str(tmp_path), measure=fake)
        assert result == {"node": 1, "rates_gbs": {"0": 20.0, "1": 50.0}}
        assert seen == [[cpus[0]], [cpus[1]]]
        assert sorted(os.sched_getaffinity(0)) == [cpus[1]]
        os.sched_setaffinity(0, before)
        flat = bind_to_fastest_upload_node(0, sysfs_root=str(tmp_path), measure=lambda d, n: 40.0)
        assert flat["node"] is None and os.sched_getaffinity(0) == before  # no clear winner: affinity restored
    finally:
        os.sched_setaffinity(0, before)
