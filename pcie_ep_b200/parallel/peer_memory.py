"""Collective set-up and tear-down of the symmetric segments.

``open_segments`` gives every rank a table of base pointers -- one per EP rank, valid on this rank's
GPU -- by one of two substrates:

``peer``
    each rank ``cudaMalloc``s its segment and exports it with CUDA IPC; the 64-byte handles are
    all-gathered over the gloo control group and every rank maps every peer (NVLink / NVSwitch).
``host_staged``
    rank 0 creates one file per rank in a private ``/dev/shm`` directory, each owner first-touches its
    own file (NUMA-bound to its GPU where the kernel allows), then every rank maps and registers all
    files with ``cudaHostRegister`` -- the reference's substrate
    (``pcie_ep/comm.py:102-234``, ``csrc/comm/advanced_shared_memory.hpp:143-288``).

Tear-down order (``Segments.close``): the caller has drained its streams and passed a barrier; peers'
mappings are released first, a second barrier follows, and only then each owner frees its memory.
"""

from __future__ import annotations

import os
from typing import Any, List, Optional

import torch.distributed as dist

from . import control


class Segments:
    """Owner of this rank's segment and of its mappings of the peers' segments."""

    def __init__(self, transport: str, rank: int, num_ranks: int, size_bytes: int, device: int) -> None:
        self.transport = transport
        self.rank = rank
        self.num_ranks = num_ranks
        self.size_bytes = size_bytes
        self.device = device
        self.pointers: List[int] = [0] * num_ranks
        self.directory: Optional[str] = None
        self.numa_bound: Optional[bool] = None
        self._own_ptr = 0
        self._imported: List[int] = []
        self._host: List[Any] = []
        self.host_pointers: List[int] = [0] * num_ranks      # host addresses of every rank's real segment
        self.outbox_host_pointers: List[int] = [0] * num_ranks  # relay mode: host addresses of this rank's outboxes
        self.relay = False
        self._closed = False

    def close(self, control_group: Any, extension: Any) -> None:
        """Collective.  Never frees memory a peer may still have mapped."""
        if self._closed:
            return
        error = None
        try:
            for ptr in self._imported:
                extension.release_imported_segment(ptr)
            self._imported = []
            kept = [seg for seg in self._host if not seg.close()]
            if kept:
                error = f"rank {self.rank}: {len(kept)} host mappings could not be unregistered and are kept"
            self._host = kept
        except Exception as exc:  # noqa: BLE001
            error = f"rank {self.rank}: {type(exc).__name__}: {exc}"
        errors = [e for e in control.gather_objects(error, control_group) if e]
        if errors:
            # a peer may still map our memory: keep it
            self._closed = True
            raise RuntimeError(f"segment release failed, memory retained: {errors}")
        if self._own_ptr:
            extension.free_device_segment(self._own_ptr)
            self._own_ptr = 0
        dist.barrier(group=control_group)
        if self.rank == 0:
            control.remove_shared_directory(self.directory)
        self._closed = True


def open_segments(
    extension: Any,
    transport: str,
    rank: int,
    num_ranks: int,
    size_bytes: int,
    device: int,
    control_group: Any,
    directory: Optional[str] = None,
    relay: bool = False,
) -> Segments:
    """Collective: allocate, exchange and map the segments of every rank.

    With ``relay`` (host-staged only) every rank additionally owns one *outbox* per peer, laid out like
    a segment; its GPU writes there instead of into the peer's segment and CPU threads forward the
    contents (``csrc/comm/numa_relay.hpp``).  The pointer table then holds the outboxes for the peers.
    """
    segments = Segments(transport, rank, num_ranks, size_bytes, device)
    segments.relay = relay
    if relay and transport != "host_staged":
        raise ValueError("relay needs the host_staged transport")
    if transport == "peer":
        def allocate() -> bytes:
            segments._own_ptr = extension.allocate_device_segment(size_bytes, device)
            return extension.export_device_segment(segments._own_ptr)

        handle = control.run_agreed(allocate, control_group, "segment allocation", rank)
        handles = control.gather_objects((os.getpid(), handle), control_group)

        def map_peers() -> None:
            for peer, (pid, peer_handle) in enumerate(handles):
                if peer == rank or pid == os.getpid() and peer_handle == handle:
                    segments.pointers[peer] = segments._own_ptr
                else:
                    ptr = extension.import_device_segment(peer_handle, device)
                    segments._imported.append(ptr)
                    segments.pointers[peer] = ptr

        control.run_agreed(map_peers, control_group, "peer mapping", rank)
    elif transport == "host_staged":
        segments.directory, _ = control.create_shared_directory(rank, control_group, directory)
        paths = [os.path.join(segments.directory, f"source-{peer}") for peer in range(num_ranks)]

        outbox_paths = [os.path.join(segments.directory, f"relay-{rank}-{peer}") for peer in range(num_ranks)]

        def create() -> None:
            if rank == 0:
                for path in paths:
                    extension.create_host_segment(path, size_bytes)
            if relay:
                for peer, path in enumerate(outbox_paths):
                    if peer != rank:
                        extension.create_host_segment(path, size_bytes)

        control.run_agreed(create, control_group, "segment creation", rank)

        def first_touch() -> None:
            node = extension.get_device_numa_node(device)
            segments.numa_bound = extension.first_touch_host_segment(paths[rank], size_bytes, node)
            if relay:
                for peer, path in enumerate(outbox_paths):
                    if peer != rank:
                        extension.first_touch_host_segment(path, size_bytes, node)

        # every owner places and touches its pages before anybody registers them
        control.run_agreed(first_touch, control_group, "first touch", rank)

        def register() -> None:
            for peer, path in enumerate(paths):
                seg = extension.HostSegment(path, size_bytes, device)
                segments._host.append(seg)
                segments.pointers[peer] = seg.device_pointer()
                segments.host_pointers[peer] = seg.host_pointer()
            if relay:
                for peer, path in enumerate(outbox_paths):
                    if peer == rank:
                        continue
                    box = extension.HostSegment(path, size_bytes, device)
                    segments._host.append(box)
                    segments.pointers[peer] = box.device_pointer()  # the GPU writes to its own outbox
                    segments.outbox_host_pointers[peer] = box.host_pointer()

        control.run_agreed(register, control_group, "host registration", rank)
    else:
        raise ValueError(f"unknown GPU transport {transport!r}")
    dist.barrier(group=control_group)
    return segments
