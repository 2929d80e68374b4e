"""Observability counters and topology discovery (fake sysfs / procfs trees, no hardware)."""
import threading

import pytest

from dlslime_b200 import _slime_c as c


@pytest.fixture(autouse=True)
def _obs_on():
    c.obs_set_enabled_for_test(True)
    c.obs_reset_for_test()
    yield
    c.obs_reset_for_test()


def test_snapshot_schema_and_once_only_accounting():
    link = c.obs_register_link("nvlink:cuda:0->cuda:1", "nvlink")
    c.obs_record_submit(link, 1, 4, 4096)  # op 1 = write
    snap = c.obs_snapshot()
    assert snap["enabled"] and snap["summary"]["pending_ops"] == 1 and snap["summary"]["pending_by_op"]["write"] == 1
    c.obs_record_complete(link, 1, 4096)
    snap = c.obs_snapshot()
    s = snap["summary"]
    for key in ("assign_total", "batch_total", "submitted_bytes_total", "completed_bytes_total", "failed_bytes_total", "pending_ops",
                "error_total", "user_mr_count", "user_mr_bytes", "sys_mr_count", "sys_mr_bytes", "mr_count", "mr_bytes", "pending_by_op"):
        assert key in s
    assert (s["assign_total"], s["batch_total"], s["completed_bytes_total"], s["pending_ops"]) == (4, 1, 4096, 0)
    nic = snap["nics"][0]
    assert nic["nic"].startswith("nvlink") and nic["kind"] == "nvlink" and nic["by_op"]["write"]["completed_bytes"] == 4096
    assert all(v >= 0 for v in s["pending_by_op"].values())


def test_register_link_is_race_free_and_deduplicated():
    slots = []
    ts = [threading.Thread(target=lambda: slots.append(c.obs_register_link("mlx5_0"))) for _ in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert len(set(slots)) == 1 and len(c.obs_snapshot()["nics"]) == 1


def test_disabled_snapshot():
    c.obs_set_enabled_for_test(False)
    assert c.obs_snapshot() == {"enabled": False} and c.obs_register_link("x") == -1


def test_system_regions_are_accounted_separately():
    import ctypes

    pool = c.MemoryPool()
    b = ctypes.create_string_buffer(1024)
    pool.register_memory_region(ctypes.addressof(b), 512, "sys.io_dummy")
    pool.register_memory_region(ctypes.addressof(b) + 512, 256, "user")
    s = c.obs_snapshot()["summary"]
    assert (s["sys_mr_count"], s["sys_mr_bytes"], s["user_mr_count"], s["user_mr_bytes"]) == (1, 512, 1, 256)


def _fake_nic(root, name, bdf, state, layer, mtu, numa):
    port = root / "class" / "infiniband" / name / "ports" / "1"
    pci = root / "devices" / "pci0000:00" / bdf
    port.mkdir(parents=True)
    pci.mkdir(parents=True)
    (port / "state").write_text(state)
    (port / "link_layer").write_text(layer)
    (port / "active_mtu").write_text(str(mtu))
    (pci / "numa_node").write_text(str(numa))
    (root / "class" / "infiniband" / name / "device").symlink_to(pci, target_is_directory=True)


def test_topology_from_fake_sysfs(tmp_path):
    _fake_nic(tmp_path, "mlx5_0", "0000:18:00.0", "4: ACTIVE\n", "Ethernet\n", 4096, 0)
    _fake_nic(tmp_path, "mlx5_1", "0000:19:00.0", "1: DOWN\n", "InfiniBand\n", 2048, 1)
    gpus = tmp_path / "proc" / "driver" / "nvidia" / "gpus" / "0000:1b:00.0"
    gpus.mkdir(parents=True)
    (gpus / "information").write_text("Model: \t NVIDIA B200\nGPU UUID: \t GPU-abc\n")
    res = c.discover_topology(preferred_device="mlx5_0", sysfs_root=str(tmp_path), devices=["mlx5_1", "mlx5_0"], procfs_root=str(tmp_path / "proc"))
    assert res["schema_version"] == 1 and res["host"]["hostname"] and res["host"]["address"] and res["memory_keys"] == []
    assert [n["name"] for n in res["nics"]] == ["mlx5_0", "mlx5_1"]
    n0, n1 = res["nics"]
    assert (n0["health"], n0["numa_node"], n0["pci_bus_id"]) == ("AVAILABLE", 0, "0000:18:00.0")
    assert n0["ports"] == [{"port": 1, "state": "ACTIVE", "link_type": "RoCE", "active_mtu": 4096}]
    assert n1["health"] == "DEGRADED" and n1["ports"][0]["link_type"] == "IB" and n1["ports"][0]["state"] == "DOWN"
    assert res["accelerators"] == [{"ordinal": 0, "pci_bus_id": "0000:1b:00.0", "kind": "cuda", "link_type": "NVLink", "model": "NVIDIA B200", "uuid": "GPU-abc"}]


def test_topology_fallbacks(tmp_path):
    res = c.discover_topology(preferred_link_type="RoCE", sysfs_root=str(tmp_path), devices=["mlx5_0"], procfs_root=str(tmp_path))
    assert res["nics"][0]["ports"] == [{"port": 1, "state": "ACTIVE", "link_type": "RoCE"}]
    res = c.discover_topology(preferred_device="hidden", preferred_link_type="RoCE", sysfs_root=str(tmp_path), devices=["mlx5_0"], procfs_root=str(tmp_path))
    assert [n["name"] for n in res["nics"]] == ["mlx5_0"]
    with pytest.raises(RuntimeError, match="No RDMA devices available"):
        c.discover_topology(sysfs_root=str(tmp_path), procfs_root=str(tmp_path))
    soft = c.discover_topology(sysfs_root=str(tmp_path), procfs_root=str(tmp_path), allow_software_links=True)
    assert soft["nics"][0]["name"] == "tcp0" and soft["nics"][0]["ports"][0]["link_type"] == "TCP"
