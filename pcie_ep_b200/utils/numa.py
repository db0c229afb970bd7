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
