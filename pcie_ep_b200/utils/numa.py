"""Host-side NUMA placement for the process that feeds one GPU.

A rank that uploads its step inputs from pinned host memory gets the full PCIe rate only when that
memory (and the thread that issues the copies) sits on the NUMA node the GPU hangs off; with eight
ranks on a two-socket machine the default placement puts most of them on the wrong socket.
``bind_to_device_numa_node`` restricts the calling process to the CPUs of the GPU's node, so that
memory it allocates afterwards (first touch, which is also where ``pin_memory`` allocates) is local.
The reference binds its host segments with ``mbind`` to the node it reads from
``/sys/bus/pci/devices/<bdf>/numa_node`` (reference: ``csrc/comm/advanced_shared_memory.hpp:120-131``);
this is the same placement decision made for the whole feeding process.
"""

from __future__ import annotations

import os
from typing import List, Optional


def parse_cpu_list(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]`` (the kernel's cpulist format)."""
    cpus: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            first, last = part.split("-", 1)
            cpus.extend(range(int(first), int(last) + 1))
        else:
            cpus.append(int(part))
    return sorted(set(cpus))


def node_cpus(node: int, sysfs_root: str = "/sys/devices/system/node") -> List[int]:
    """CPUs of one NUMA node, empty when the node (or sysfs) is not there."""
    try:
        with open(os.path.join(sysfs_root, f"node{node}", "cpulist")) as handle:
            return parse_cpu_list(handle.read())
    except (OSError, ValueError):
        return []


def bind_to_device_numa_node(device: int, numa_node: Optional[int] = None,
                             sysfs_root: str = "/sys/devices/system/node") -> Optional[int]:
    """Restrict this process to the CPUs of ``device``'s NUMA node.

    Returns the node it bound to, or ``None`` when nothing was changed (node unknown, a single node,
    no permitted CPU on that node).  ``numa_node`` overrides the look-up (tests)."""
    if numa_node is None:
        from .. import _C

        numa_node = int(_C.get_device_numa_node(device))
    if numa_node < 0:
        return None
    cpus = node_cpus(numa_node, sysfs_root)
    if not cpus:
        return None
    try:
        allowed = os.sched_getaffinity(0)
        target = allowed.intersection(cpus)
        if not target or target == allowed:
            return None if not target else numa_node
        os.sched_setaffinity(0, target)
    except (AttributeError, OSError):
        return None
    return numa_node


def available_nodes(sysfs_root: str = "/sys/devices/system/node") -> List[int]:
    """NUMA nodes that own at least one CPU this process may run on."""
    try:
        allowed = os.sched_getaffinity(0)
        names = sorted(os.listdir(sysfs_root))
    except (AttributeError, OSError):
        return []
    nodes = []
    for name in names:
        if name.startswith("node") and name[4:].isdigit() and allowed.intersection(node_cpus(int(name[4:]), sysfs_root)):
            nodes.append(int(name[4:]))
    return sorted(nodes)


def measure_upload_rate(device: int, num_bytes: int, repeats: int = 3) -> float:
    """GB/s of a pinned-host -> device copy issued by this thread with memory it allocates now."""
    import torch

    host = torch.empty(num_bytes, dtype=torch.uint8, pin_memory=True)
    host.fill_(1)
    target = torch.empty(num_bytes, dtype=torch.uint8, device=torch.device("cuda", device))
    target.copy_(host, non_blocking=True)
    torch.cuda.synchronize(device)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        target.copy_(host, non_blocking=True)
    stop.record()
    stop.synchronize()
    _PROBE_BUFFERS.append(host)  # a freed pinned block would be handed to the next node's probe
    return repeats * num_bytes / (start.elapsed_time(stop) * 1e-3) / 1e9


#: pinned probe buffers kept alive until a placement decision is complete
_PROBE_BUFFERS: List[object] = []


def bind_to_fastest_upload_node(device: int, probe_bytes: int = 48 << 20, min_gain: float = 1.05,
                                sysfs_root: str = "/sys/devices/system/node", measure=None) -> Optional[dict]:
    """Where the platform does not say which NUMA node a GPU hangs off (``numa_node`` reads -1 in many
    virtualised hosts), find out by measurement: from the CPUs of every node in turn, allocate pinned memory
    and time a host -> device copy; stay on the node with the highest rate when it beats the slowest by
    ``min_gain``, otherwise restore the original affinity.  Call it while no other rank is copying (ranks take
    turns).  Returns ``{"node": chosen or None, "rates_gbs": {node: rate}}``, or ``None`` with fewer than two nodes.
    ``measure(device, num_bytes)`` replaces the CUDA probe in tests."""
    nodes = available_nodes(sysfs_root)
    if len(nodes) < 2:
        return None
    measure = measure or measure_upload_rate
    original = os.sched_getaffinity(0)
    rates = {}
    try:
        for position, node in enumerate(nodes):
            os.sched_setaffinity(0, original.intersection(node_cpus(node, sysfs_root)))
            rates[node] = float(measure(device, probe_bytes + position * (4 << 20)))  # growing sizes: no cached block fits
        best = max(rates, key=rates.get)
        if rates[best] >= min_gain * min(rates.values()):
            os.sched_setaffinity(0, original.intersection(node_cpus(best, sysfs_root)))
            chosen: Optional[int] = best
        else:
            os.sched_setaffinity(0, original)
            chosen = None
    except OSError:
        os.sched_setaffinity(0, original)
        return None
    finally:
        _PROBE_BUFFERS.clear()
    return {"node": chosen, "rates_gbs": {str(k): round(v, 1) for k, v in rates.items()}}
