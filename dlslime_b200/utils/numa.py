"""NUMA placement of a rank next to its GPU (or NIC).

Pinned host buffers are allocated on the NUMA node of the thread that touches them first; a rank whose thread runs on
the other socket pays the inter-socket link on every host<->device copy. ``bind_to_device_numa`` restricts the
calling process to the cores of the node its GPU hangs off, so that staging buffers allocated afterwards are local.
Role in the reference: ``bindToSocket`` / ``socketId`` for NICs (``dlslime/csrc/engine/rdma/rdma_utils.h:26-122`` in the
reference); here for GPUs as well, and without libnuma (sysfs + ``sched_setaffinity``).
"""

from __future__ import annotations

import os


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def node_cpus(node: int, sysfs_root: str = "/sys") -> set[int]:
    try:
        with open(os.path.join(sysfs_root, "devices/system/node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read())
    except OSError:
        return set()


def pci_numa_node(bus_id: str, sysfs_root: str = "/sys") -> int:
    """NUMA node of a PCI function given as ``dddd:bb:dd.f`` (case-insensitive); -1 when unknown."""
    try:
        with open(os.path.join(sysfs_root, "bus/pci/devices", bus_id.lower(), "numa_node")) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return -1


def device_pci_bus_id(index: int) -> str | None:
    try:
        import torch

        p = torch.cuda.get_device_properties(index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        pass
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        return bus[-12:].lower()  # NVML prints an 8-digit domain
    except Exception:
        return None


def device_numa_node(index: int, sysfs_root: str = "/sys") -> int:
    bus = device_pci_bus_id(index)
    return pci_numa_node(bus, sysfs_root) if bus else -1


def bind_to_numa_node(node: int, sysfs_root: str = "/sys") -> bool:
    cpus = node_cpus(node, sysfs_root)
    if node < 0 or not cpus:
        return False
    try:
        allowed = os.sched_getaffinity(0)
        target = cpus & allowed or cpus
        os.sched_setaffinity(0, target)
        return True
    except OSError:
        return False


def bind_to_device_numa(index: int, sysfs_root: str = "/sys") -> int:
    """Pin the calling process to the NUMA node of CUDA device ``index``. Returns the node, or -1 if nothing was done."""
    node = device_numa_node(index, sysfs_root)
    return node if bind_to_numa_node(node, sysfs_root) else -1
