"""What a dispatch leaves behind: the handle of one result and the detachable routing cache.

Parity: the reference's ``pcie_ep/buffers/handle.py:15-174`` (same attribute names, including the
DeepEP aliases, and the same set of cached-layout rejections).  Every count lives on the device and is
never read back by the library; ``check_errors`` is the one explicit synchronising call.
"""

from __future__ import annotations

from typing import Any, Dict, Optional, TYPE_CHECKING

import torch

from ..utils.event import EventOverlap

if TYPE_CHECKING:  # pragma: no cover
    from .ep import HostStagedEPBuffer


def _fingerprint(tensor: torch.Tensor) -> tuple:
    """Everything that makes a tensor 'the same memory seen the same way' (not its contents)."""
    return (id(tensor), tensor.data_ptr(), tuple(tensor.shape), tuple(tensor.stride()), tensor.dtype, tensor.device)


class RouteBinding:
    """The routing tensor a plan was computed from, with the means to notice that it changed.

    PyTorch bumps a tensor's version counter on every in-place write; inference tensors have none,
    which is why they can be dispatched but not cached.
    """

    __slots__ = ("tensor", "version", "fingerprint")

    def __init__(self, tensor: torch.Tensor) -> None:
        self.tensor = tensor
        self.version: Optional[int] = None if tensor.is_inference() else tensor._version
        self.fingerprint = _fingerprint(tensor)

    @property
    def cacheable(self) -> bool:
        return self.version is not None

    def current(self) -> torch.Tensor:
        if self.version is not None and self.tensor._version != self.version:
            raise RuntimeError("topk_idx changed after the dispatch that this handle describes; dispatch again instead of reusing it")
        return self.tensor

    def same_memory(self) -> bool:
        return _fingerprint(self.tensor) == self.fingerprint


class _Routed:
    """What the handle and the cached layout have in common: a routing tensor and the buffer state it is valid for."""

    _route: RouteBinding
    _layout: Any
    _owner: Any

    @property
    def topk_idx(self) -> torch.Tensor:
        return self._route.current()

    # kept for callers that looked at these directly
    @property
    def _topk_version(self) -> Optional[int]:
        return self._route.version

    def validate_cached(self, owner: "HostStagedEPBuffer", x: torch.Tensor, alignment: int, do_expand: bool) -> Any:
        """May this routing be reused for ``x`` on ``owner``?  Returns the native plan.  Host-side checks only."""
        if (self.buffer_id, self.generation) != (owner.buffer_id, owner._generation):
            raise ValueError("cached routing was produced by another buffer, or the buffer has been rebuilt since")
        if self._owner is not owner or self.group is not owner.group or self.global_ranks != owner.global_ranks:
            raise ValueError("cached routing belongs to a different EP group or rank-to-expert ownership")
        if (self.num_experts, self.num_max_tokens_per_rank) != (owner.num_experts, owner.num_max_tokens_per_rank):
            raise ValueError("cached routing was made for other buffer dimensions")
        route = self.topk_idx  # raises if the routing tensor was written to
        if not self._route.cacheable:
            raise ValueError("a routing tensor without a PyTorch version counter (inference tensor) cannot be cached")
        if not self._route.same_memory():
            raise ValueError("the cached routing tensor now has another address, shape or stride")
        if tuple(x.shape) != (route.shape[0], owner.hidden):
            raise ValueError(f"x has shape {tuple(x.shape)}, the cached routing covers {route.shape[0]} tokens of hidden {owner.hidden}")
        if (alignment, bool(do_expand)) != (self.expert_alignment, bool(self.do_expand)):
            raise ValueError("a cached routing fixes expert alignment and layout: alignment or expansion differs from the cached dispatch")
        if self._layout is None:
            raise RuntimeError("this dispatch produced no reusable native routing plan")
        return self._layout


# attribute on the handle -> key of the native result (DeepEP-compatible aliases included)
_RESULT_FIELDS = {
    "unique_count": "unique_count",
    "num_recv_tokens": "unique_count",
    "expanded_count": "expanded_count",
    "num_expanded_tokens": "expanded_count",
    "expert_counts": "expert_counts",
    "num_unaligned_recv_tokens_per_expert": "expert_counts",
    "expert_offsets": "expert_offsets",
    "psum_num_recv_tokens_per_expert": "expert_prefix",
    "source_meta": "source_meta",
    "recv_src_metadata": "source_meta",
    "source_offsets": "source_offsets",
    "source_expert_prefix": "source_expert_prefix",
    "error": "error",
    "stats": "stats",
    "transport_timestamps_ns": "transport_timestamps_ns",
    "prefix_tx_timestamps_ns": "prefix_tx_timestamps_ns",
    "receive_expand_overlap": "receive_expand_overlap",
    "profiling": "profiling",
    "role_profiling": "role_profiling",
    "dst_buffer_slot_idx": "dst_buffer_slot_idx",
}


class HostStagedEPHandle(_Routed):
    """Device-side description of one capacity-shaped dispatch result.

    Result tensors are looked up in the native result when first asked for, so a dispatch spends no CPU
    time on fields nobody reads.
    """

    def __init__(self, owner: "HostStagedEPBuffer", topk_idx: torch.Tensor, result: Dict[str, Any], do_expand: bool,
                 expert_alignment: int, event: EventOverlap) -> None:
        self._owner = owner
        self._route = RouteBinding(topk_idx)
        self._result = result
        self._layout = result.get("_layout")
        self.buffer_id, self.generation = owner.buffer_id, owner._generation
        self.group, self.global_ranks = owner.group, owner.global_ranks
        self.num_experts, self.num_max_tokens_per_rank = owner.num_experts, owner.num_max_tokens_per_rank
        self.do_expand, self.expert_alignment = do_expand, expert_alignment
        self.num_sms = 0
        self.num_recv_tokens_per_expert_list = None
        self.completion = event
        self._completion_event = event.event

    def __getattr__(self, name: str) -> Any:
        # reached only for names that __init__ did not set: resolve against the native result and remember
        if name == "psum_num_recv_tokens_per_scaleup_rank":
            value = self._result["source_offsets"][1:]
        else:
            key = _RESULT_FIELDS.get(name)
            if key is None:
                raise AttributeError(name)
            value = self._result.get(key)
        self.__dict__[name] = value
        return value

    def check_errors(self) -> None:
        """Explicit diagnostic: waits for this dispatch and raises if the device recorded an error."""
        self._owner.check_errors(self)

    def cache_layout(self) -> "CachedLayout":
        return CachedLayout(self)

    @property
    def cached_layout(self) -> "CachedLayout":
        return CachedLayout(self)


class CachedLayout(_Routed):
    """A routing plan detached from its result: holds the routing tensor's identity and the native plan, and
    no output tensor, so keeping it alive does not keep a result pool busy."""

    _COPIED = ("_owner", "_layout", "buffer_id", "generation", "group", "global_ranks", "num_experts",
               "num_max_tokens_per_rank", "expert_alignment", "do_expand")

    def __init__(self, handle: HostStagedEPHandle) -> None:
        if handle._layout is None:
            raise RuntimeError("this dispatch produced no reusable native routing plan")
        if not handle._route.cacheable:
            raise ValueError("a routing tensor without a PyTorch version counter (inference tensor) cannot be cached")
        handle.topk_idx  # refuses a routing tensor that has been written to since
        self._route = handle._route
        for name in self._COPIED:
            setattr(self, name, getattr(handle, name))


EPHandle = HostStagedEPHandle
