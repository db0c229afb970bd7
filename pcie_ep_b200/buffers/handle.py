"""Result handle of one dispatch and the detachable routing cache.

Field names (including the DeepEP aliases) follow the reference's handle
(``pcie_ep/buffers/handle.py:55-111``).  All counts live on the device and are never read back by
the library; ``check_errors`` is the one explicit synchronising call.
"""

from __future__ import annotations

from typing import Any, Dict, Optional, TYPE_CHECKING

import torch

from ..utils.event import EventOverlap

if TYPE_CHECKING:  # pragma: no cover
    from .ep import HostStagedEPBuffer


def _tensor_signature(tensor: torch.Tensor) -> tuple:
    return (id(tensor), tensor.data_ptr(), tuple(tensor.shape), tuple(tensor.stride()), tensor.dtype, tensor.device)


class _RouteGuard:
    """Shared by the handle and the cached layout: the routing tensor must not change under them."""

    _topk_idx: torch.Tensor
    _topk_version: Optional[int]
    _route_signature: tuple

    @property
    def topk_idx(self) -> torch.Tensor:
        if self._topk_version is not None and self._topk_idx._version != self._topk_version:
            raise RuntimeError("topk_idx changed while its dispatch handle was in use")
        return self._topk_idx

    def validate_cached(self, owner: "HostStagedEPBuffer", x: torch.Tensor, alignment: int, do_expand: bool) -> Any:
        """Host-side checks only; no device value is read (reference: ``handle.py:117-136``)."""
        if self.buffer_id != owner.buffer_id or self.generation != owner._generation:
            raise ValueError("Cached handle belongs to another buffer generation")
        if self._owner is not owner or self.group is not owner.group or self.global_ranks != owner.global_ranks:
            raise ValueError("Cached handle belongs to another EP group or owner map")
        if self.num_experts != owner.num_experts or self.num_max_tokens_per_rank != owner.num_max_tokens_per_rank:
            raise ValueError("Cached handle dimensions or expert ownership changed")
        route = self.topk_idx
        if self._topk_version is None:
            raise ValueError("Cached routing requires a tensor with a PyTorch version counter")
        if _tensor_signature(route) != self._route_signature:
            raise ValueError("Cached routing tensor address, shape or strides changed")
        if x.shape[0] != route.shape[0] or x.shape[1] != owner.hidden:
            raise ValueError("Cached dispatch input dimensions changed")
        if (alignment, do_expand) != (self.expert_alignment, self.do_expand):
            raise ValueError("Cached dispatch alignment or expansion mode changed")
        if self._layout is None:
            raise RuntimeError("The native runtime did not provide an immutable cached layout")
        return self._layout


class HostStagedEPHandle(_RouteGuard):
    """Device-side description of one capacity-shaped dispatch result."""

    def __init__(
        self,
        owner: "HostStagedEPBuffer",
        topk_idx: torch.Tensor,
        result: Dict[str, Any],
        do_expand: bool,
        expert_alignment: int,
        event: EventOverlap,
    ) -> None:
        self.buffer_id = owner.buffer_id
        self.generation = owner._generation
        self.group = owner.group
        self.global_ranks = owner.global_ranks
        self.do_expand = do_expand
        self.expert_alignment = expert_alignment
        self.num_experts = owner.num_experts
        self.num_max_tokens_per_rank = owner.num_max_tokens_per_rank
        self.num_sms = 0
        self._topk_idx = topk_idx
        self._topk_version = None if topk_idx.is_inference() else topk_idx._version
        self._route_signature = _tensor_signature(topk_idx)
        self._layout = result.get("_layout")
        self._result = result
        self.num_recv_tokens_per_expert_list = None
        self.completion = event
        self._completion_event = event.event
        self._owner = owner

    # Result fields are looked up when first asked for (a dispatch touches none of them on the CPU).
    # name on the handle -> key in the native result; DeepEP-compatible aliases included.
    _FIELDS = {
        "unique_count": "unique_count",
        "num_recv_tokens": "unique_count",
        "expanded_count": "expanded_count",
        "num_expanded_tokens": "expanded_count",
        "expert_counts": "expert_counts",
        "num_unaligned_recv_tokens_per_expert": "expert_counts",
        "expert_offsets": "expert_offsets",
        "source_meta": "source_meta",
        "recv_src_metadata": "source_meta",
        "source_offsets": "source_offsets",
        "source_expert_prefix": "source_expert_prefix",
        "psum_num_recv_tokens_per_expert": "expert_prefix",
        "error": "error",
        "stats": "stats",
        "transport_timestamps_ns": "transport_timestamps_ns",
        "receive_expand_overlap": "receive_expand_overlap",
        "prefix_tx_timestamps_ns": "prefix_tx_timestamps_ns",
        "profiling": "profiling",
        "dst_buffer_slot_idx": "dst_buffer_slot_idx",
    }

    def __getattr__(self, name: str) -> Any:
        # only called for attributes not set in __init__
        if name == "psum_num_recv_tokens_per_scaleup_rank":
            value = self._result["source_offsets"][1:]
        elif name in HostStagedEPHandle._FIELDS:
            value = self._result.get(HostStagedEPHandle._FIELDS[name])
        else:
            raise AttributeError(name)
        self.__dict__[name] = value
        return value

    def check_errors(self) -> None:
        """Explicit diagnostic synchronisation; never called by dispatch itself."""
        self._owner.check_errors(self)

    def cache_layout(self) -> "CachedLayout":
        return CachedLayout(self)

    @property
    def cached_layout(self) -> "CachedLayout":
        return self.cache_layout()

    _tensor_signature = staticmethod(_tensor_signature)


class CachedLayout(_RouteGuard):
    """Routing plan + route identity, without any result-pool tensor (reference: ``handle.py:139-171``)."""

    def __init__(self, handle: HostStagedEPHandle) -> None:
        if handle._layout is None:
            raise RuntimeError("This dispatch has no immutable native layout to cache")
        if handle._topk_version is None:
            raise ValueError("Cached routing requires a PyTorch version counter")
        self._topk_idx = handle.topk_idx
        for name in (
            "_topk_version", "_route_signature", "_layout", "_owner", "buffer_id", "generation", "group",
            "global_ranks", "num_experts", "num_max_tokens_per_rank", "expert_alignment", "do_expand",
        ):
            setattr(self, name, getattr(handle, name))

    _tensor_signature = staticmethod(_tensor_signature)


EPHandle = HostStagedEPHandle
