"""Control plane: everything that talks to other processes, all of it at construction or close.

The hot path never issues a collective (reference: ``pcie_ep/comm.py`` -- gloo for init and teardown
only).  Every step that can fail on one rank ends in an agreement round so that all ranks raise
together instead of some of them waiting in the next collective forever
(reference: ``pcie_ep/comm.py:185-234``).
"""

from __future__ import annotations

import os
import shutil
import socket
import tempfile
import uuid
from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..config import HostStagedConfig


@dataclass
class BorrowedNCCLComm:
    """Result of looking for the application's NCCL communicator; nothing is ever created."""

    nccl_comm: Optional[int]
    reused: bool
    status: str
    group: Any = None


def borrow_nccl_comm(group: Any, device: Any, require_reuse: bool = False) -> BorrowedNCCLComm:
    """Read the raw communicator of an NCCL group if PyTorch exposes it.

    The transport issues no NCCL call; the pointer is only recorded so an application can check
    that no second communicator was made.
    """
    try:
        backend_name = dist.get_backend(group)
    except Exception:  # pragma: no cover - uninitialised group
        backend_name = "unknown"
    if "nccl" not in str(backend_name):
        if require_reuse:
            raise RuntimeError("require_reuse_nccl_comm=True needs an NCCL process group")
        return BorrowedNCCLComm(None, False, "not_an_nccl_group")
    try:
        torch_device = torch.device("cuda", device) if isinstance(device, int) else device
        backend = group._get_backend(torch_device)
        pointer = backend._comm_ptr()
        return BorrowedNCCLComm(int(pointer), True, "reused", group)
    except Exception as exc:
        if require_reuse:
            raise RuntimeError(f"cannot borrow the NCCL communicator: {exc}") from exc
        return BorrowedNCCLComm(None, False, f"unavailable: {type(exc).__name__}", group)


def get_control_group(group: Any, global_ranks: Sequence[int], control_group: Any = None) -> Tuple[Any, bool]:
    """Return ``(gloo group with the same ordered members, whether this call created it)``."""
    if control_group is not None:
        if "gloo" not in str(dist.get_backend(control_group)):
            raise ValueError("control_group must be a gloo group")
        if tuple(dist.get_process_group_ranks(control_group)) != tuple(global_ranks):
            raise ValueError("control_group must have the same ordered ranks as the EP group")
        return control_group, False
    if "gloo" in str(dist.get_backend(group)):
        return group, False
    return dist.new_group(ranks=list(global_ranks), backend="gloo"), True


def gather_objects(value: Any, group: Any) -> List[Any]:
    values: List[Any] = [None] * dist.get_world_size(group)
    dist.all_gather_object(values, value, group=group)
    return values


def agree(error: Optional[str], group: Any, what: str) -> None:
    """Collective: raise on every rank if any rank reports an error."""
    errors = [e for e in gather_objects(error, group) if e]
    if errors:
        raise RuntimeError(f"{what} failed: {errors}")


def run_agreed(step: Callable[[], Any], group: Any, what: str, rank: int) -> Any:
    """Run ``step`` locally, then agree on success; returns the local result."""
    result, error = None, None
    try:
        result = step()
    except Exception as exc:  # noqa: BLE001 - reported collectively
        error = f"rank {rank}: {type(exc).__name__}: {exc}"
    agree(error, group, what)
    return result


def validate_group_configuration(
    control_group: Any,
    num_ranks: int,
    num_max_tokens_per_rank: int,
    hidden: int,
    num_topk: int,
    num_experts: int,
    config: HostStagedConfig,
    transport: str,
    require_same_host: bool = True,
) -> None:
    """All ranks must run on one host with identical dimensions and options."""
    mine = (
        socket.gethostname() if require_same_host else "",
        (num_ranks, num_max_tokens_per_rank, hidden, num_topk, num_experts),
        tuple(sorted((k, str(v)) for k, v in config.native_options().items())),
        transport,
    )
    everyone = gather_objects(mine, control_group)
    if any(other != everyone[0] for other in everyone):
        raise RuntimeError("EP ranks disagree on host, dimensions, transport or configuration")


def create_shared_directory(rank: int, control_group: Any, parent: Optional[str]) -> Tuple[str, str]:
    """Rank 0 makes a private directory (``/dev/shm`` by default) and tells the others."""
    payload = [None]
    error = None
    if rank == 0:
        try:
            base = parent or ("/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir())
            directory = tempfile.mkdtemp(prefix="pcie-ep-b200-", dir=base)
            payload = [{"directory": directory, "id": uuid.uuid4().hex}]
        except Exception as exc:  # noqa: BLE001
            error = f"rank 0: {type(exc).__name__}: {exc}"
            payload = [{"error": error}]
    dist.broadcast_object_list(payload, src=dist.get_global_rank(control_group, 0), group=control_group)
    info = payload[0]
    if "error" in info:
        raise RuntimeError(f"creating the shared directory failed: {info['error']}")
    return info["directory"], info["id"]


def remove_shared_directory(directory: Optional[str]) -> None:
    if directory and os.path.isdir(directory):
        shutil.rmtree(directory, ignore_errors=True)
