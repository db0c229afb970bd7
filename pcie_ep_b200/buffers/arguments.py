"""Argument checking shared by ``dispatch``, ``capture_dispatch`` and ``combine``.

Everything here runs on the host and reads no device value.  The rules are kept as data (tables of
names and messages, tensor rules with wildcard shapes) so that the eager and the graph entry points
cannot drift apart.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Sequence, Tuple

import torch

MAX_ALIGNMENT = 256

# DeepEP keywords this library accepts for source compatibility but does not implement: keyword -> why
UNSUPPORTED_DISPATCH_KEYWORDS = (
    ("do_cpu_sync", "dispatch never waits on the CPU; sizes stay on the device (do_cpu_sync must be False)"),
    ("do_handle_copy", "handles are not copied; cache_layout() detaches a routing plan instead"),
    ("num_qps", "there are no queue pairs on this transport"),
    ("num_sms", "the dispatch grid is fixed by the buffer's channel count; num_sms cannot override it"),
    ("use_tma_aligned_col_major_sf", "scale factors are one FP32 per row; no column-major layout exists"),
)


@dataclass(frozen=True)
class TensorRule:
    """What one tensor argument must look like.  ``dtype=None`` accepts any floating type; ``None`` in
    ``shape`` matches any extent."""

    name: str
    dtype: Optional[torch.dtype]
    shape: Tuple[Optional[int], ...]

    def check(self, value: Any, *, device: Any, on_gpu: bool) -> None:
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{self.name}: expected a torch.Tensor, got {type(value).__name__}")
        if on_gpu:
            if not value.is_cuda or value.device.index != device:
                raise ValueError(f"{self.name}: tensor lives on {value.device}, the buffer on cuda:{device}")
        elif value.is_cuda:
            raise ValueError(f"{self.name}: the cpu transport takes CPU tensors, got one on {value.device}")
        if self.dtype is None:
            if not value.is_floating_point():
                raise ValueError(f"{self.name}: expected a floating-point tensor, got {value.dtype}")
        elif value.dtype != self.dtype:
            raise ValueError(f"{self.name}: expected dtype {self.dtype}, got {value.dtype}")
        if not value.is_contiguous():
            raise ValueError(f"{self.name}: tensor must be contiguous")
        extents = tuple(value.shape)
        if len(extents) != len(self.shape) or any(want is not None and want != got for want, got in zip(self.shape, extents)):
            wanted = tuple("*" if want is None else want for want in self.shape)
            raise ValueError(f"{self.name}: shape {extents} does not fit {wanted}")


def reject_unsupported(values: dict) -> None:
    """Raise for the first accepted-but-unimplemented keyword that was actually used."""
    for keyword, why in UNSUPPORTED_DISPATCH_KEYWORDS:
        if values.get(keyword):
            raise NotImplementedError(f"{keyword}: {why}")


def resolve_alignment(requested: Any, inherited: Optional[int], upper: Optional[int] = None) -> int:
    """``expert_alignment`` as given, else the cached handle's, else 1."""
    value = requested if requested is not None else (inherited if inherited is not None else 1)
    if isinstance(value, bool) or not isinstance(value, int) or value < 1:
        raise ValueError(f"expert_alignment must be a positive integer, got {value!r}")
    if upper is not None and value > upper:
        raise ValueError(f"expert_alignment must lie in [1, {upper}], got {value}")
    return value


@dataclass
class DispatchRequest:
    """A dispatch call after validation: what the native runtime needs, nothing else."""

    x: torch.Tensor
    topk_idx: torch.Tensor
    topk_weights: Optional[torch.Tensor]
    cumulative: Optional[torch.Tensor]
    alignment: int
    expand: bool
    zero_padding: bool
    cached_layout: Any          # native routing plan of a cached handle, or None
    source_handle: Any          # the cached handle / layout itself, or None

    def keepalive(self, owner: Any, result: Any) -> Sequence[Any]:
        refs = [owner, self.x, self.topk_idx, self.topk_weights, result, self.cumulative]
        if self.source_handle is not None:
            refs.append(self.source_handle)
        return tuple(refs)


def build_dispatch_request(owner: Any, x: Any, topk_idx: Any, topk_weights: Any, *, handle: Any, expert_alignment: Any,
                           do_expand: bool, do_zero_padding: bool, cumulative: Any = None, num_experts: Any = None,
                           num_max_tokens_per_rank: Any = None, alignment_limit: Optional[int] = None) -> DispatchRequest:
    """Validate the tensor arguments of a dispatch against ``owner`` (an EP buffer)."""
    if handle is not None:
        if topk_idx is not None:
            raise ValueError("pass either topk_idx or a cached handle: the handle already names its routing tensor")
        topk_idx = handle.topk_idx
    if do_zero_padding and not do_expand:
        raise ValueError("do_zero_padding pads expert segments, which exist only with do_expand=True")
    alignment = resolve_alignment(expert_alignment, getattr(handle, "expert_alignment", None), alignment_limit)
    for name, given, prepared in (("num_experts", num_experts, owner.num_experts),
                                  ("num_max_tokens_per_rank", num_max_tokens_per_rank, owner.num_max_tokens_per_rank)):
        if given is not None and given != prepared:
            raise ValueError(f"{name}={given} contradicts the buffer, which was built for {prepared}")
    device, on_gpu = owner.device, owner.on_gpu
    TensorRule("x", torch.bfloat16 if on_gpu else None, (None, owner.hidden)).check(x, device=device, on_gpu=on_gpu)
    tokens = x.shape[0]
    if tokens > owner.num_max_tokens_per_rank:
        raise ValueError(f"x has {tokens} tokens, the buffer holds at most {owner.num_max_tokens_per_rank} per rank")
    TensorRule("topk_idx", torch.int64, (tokens, owner.num_topk)).check(topk_idx, device=device, on_gpu=on_gpu)
    if topk_weights is not None:
        TensorRule("topk_weights", torch.float32, (tokens, owner.num_topk)).check(topk_weights, device=device, on_gpu=on_gpu)
    if cumulative is not None:
        TensorRule("cumulative_local_expert_recv_stats", torch.int32, (owner.num_experts // owner.num_ranks,)).check(
            cumulative, device=device, on_gpu=on_gpu)
    cached = handle.validate_cached(owner, x, alignment, do_expand) if handle is not None else None
    return DispatchRequest(x, topk_idx, topk_weights, cumulative, alignment, bool(do_expand), bool(do_zero_padding), cached, handle)
