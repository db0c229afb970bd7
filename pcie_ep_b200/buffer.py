"""Legacy import path (reference: ``pcie_ep/buffer.py:1-27``); also the place tests patch."""

import torch
import torch.distributed as dist  # noqa: F401  (patch target)

from .buffers.ep import EPBuffer, HostStagedEPBuffer
from .buffers.handle import CachedLayout, EPHandle, HostStagedEPHandle
from .config import HostStagedConfig
from .graph import GraphDispatch
from .utils.event import EventOverlap

topk_idx_t = torch.int64

__all__ = [
    "CachedLayout", "EPBuffer", "EPHandle", "EventOverlap", "GraphDispatch", "HostStagedConfig",
    "HostStagedEPBuffer", "HostStagedEPHandle", "topk_idx_t",
]
