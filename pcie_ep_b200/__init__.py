"""Blackwell-native expert-parallel dispatch/combine with a DeepEP-shaped API.

Exports mirror the reference package (``pcie_ep/__init__.py:16-28``) so ``from pcie_ep_b200 import
HostStagedConfig, HostStagedEPBuffer`` is a drop-in replacement, plus the additions of this build
(``combine``, the MoE layer, the grouped expert FFN).
"""

import torch

from .buffers.ep import EPBuffer, HostStagedEPBuffer
from .buffers.handle import CachedLayout, EPHandle, HostStagedEPHandle
from .config import EPConfig, HostStagedConfig
from .graph import GraphDispatch
from .quantization import dequantize_fp8_reference, fp8_roundtrip_reference, quantize_fp8_reference
from .utils.event import EventOverlap

topk_idx_t = torch.int64

__all__ = [
    "CachedLayout",
    "EPBuffer",
    "EPConfig",
    "EPHandle",
    "EventOverlap",
    "GraphDispatch",
    "HostStagedConfig",
    "HostStagedEPBuffer",
    "HostStagedEPHandle",
    "dequantize_fp8_reference",
    "fp8_roundtrip_reference",
    "quantize_fp8_reference",
    "topk_idx_t",
]
