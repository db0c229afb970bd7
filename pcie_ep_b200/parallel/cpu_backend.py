"""CPU transport: the dispatch/combine semantics over a gloo group, in plain PyTorch.

It is the oracle the GPU kernels are checked against, the backend of machines without a GPU and
the timed CPU baseline.  Every rank all-gathers the inputs and evaluates
``ops.reference.dispatch_reference`` for itself, so results are bit-identical to the definition
(the reference project's tests do the same with ``all_gather_object`` and a per-token loop:
``tests/test_correctness.py:26-92``).

The class mirrors the native ``Runtime`` surface that ``EPBuffer`` uses.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import reference


class CpuLayout:
    """Routing plan of the CPU transport: the gathered routes, reusable while they do not change."""

    def __init__(self, routes: List[torch.Tensor], num_tokens: int, alignment: int, expand: bool) -> None:
        self.routes = routes
        self.num_tokens = num_tokens
        self.alignment = alignment
        self.expand = expand
        self.valid = True


class CpuRuntime:
    def __init__(
        self,
        rank: int,
        num_ranks: int,
        num_max_tokens: int,
        hidden: int,
        num_topk: int,
        num_experts: int,
        options: Dict[str, Any],
        group: Any,
    ) -> None:
        self.rank, self.num_ranks = rank, num_ranks
        self.num_max_tokens, self.hidden, self.num_topk, self.num_experts = num_max_tokens, hidden, num_topk, num_experts
        self.options = dict(options)
        self.group = group
        self.wire_dtype = self.options.get("wire_dtype", "bf16")
        self._failed = False
        self._closed = False
        self._outstanding = 0

    # -- helpers ----------------------------------------------------------------------------
    def _gather(self, value: Any) -> List[Any]:
        values: List[Any] = [None] * self.num_ranks
        dist.all_gather_object(values, value, group=self.group)
        return values

    def unique_capacity(self) -> int:
        return reference.unique_capacity(self.num_ranks, self.num_max_tokens)

    def expanded_capacity(self) -> int:
        return reference.expanded_capacity(self.num_ranks, self.num_max_tokens, self.num_topk, self.num_experts)

    # -- API used by EPBuffer ---------------------------------------------------------------
    def dispatch(
        self,
        x: torch.Tensor,
        topk_idx: torch.Tensor,
        topk_weights: Optional[torch.Tensor],
        alignment: int,
        expand: bool,
        zero_padding: bool,
        cached: Optional[CpuLayout],
        graph_pool: bool,
    ) -> Dict[str, Any]:
        if self._closed:
            raise RuntimeError("runtime is closed")
        if not 1 <= alignment <= 256:
            raise ValueError("expert_alignment must be in [1,256]")
        inputs = self._gather((x, topk_idx, topk_weights))
        ok = all(reference.validate_routes(idx, self.num_experts) for _, idx, _ in inputs)
        if not ok or self._failed:
            # invalid routing anywhere aborts every rank, like the GPU protocol does
            self._failed = True
            result = self._empty_result(x, expand)
            result["error"][0] = 2 if not ok else 19
            return result
        result = reference.dispatch_reference(
            inputs,
            self.rank,
            self.num_experts,
            self.num_max_tokens,
            do_expand=expand,
            expert_alignment=alignment,
            do_zero_padding=zero_padding,
            wire_dtype=self.wire_dtype,
        )
        result["_layout"] = cached or CpuLayout([idx for _, idx, _ in inputs], x.shape[0], alignment, expand)
        result["_expand"] = expand
        result["_num_tokens"] = x.shape[0]
        result["_all_tokens"] = [inp[0].shape[0] for inp in inputs]
        result["transport_timestamps_ns"] = torch.zeros(2, dtype=torch.int64)
        result["prefix_tx_timestamps_ns"] = None
        return result

    def _empty_result(self, x: torch.Tensor, expand: bool) -> Dict[str, Any]:
        local = self.num_experts // self.num_ranks
        cap = self.expanded_capacity() if expand else self.unique_capacity()
        shape = (cap,) if expand else (cap, self.num_topk)
        return {
            "recv_x": torch.zeros(cap, self.hidden, dtype=x.dtype),
            "recv_topk_idx": torch.full(shape, -1, dtype=torch.int64),
            "recv_topk_weights": torch.zeros(shape, dtype=torch.float32),
            "recv_topk_weights_full": torch.zeros(shape, dtype=torch.float32),
            "source_meta": torch.full((cap, 3), -1, dtype=torch.int64),
            "valid_rows": torch.zeros(cap, dtype=torch.bool),
            "unique_count": torch.zeros(1, dtype=torch.int64),
            "expanded_count": torch.zeros(1, dtype=torch.int64),
            "expert_counts": torch.zeros(local, dtype=torch.int32),
            "expert_offsets": torch.zeros(local + 1, dtype=torch.int32),
            "expert_prefix": torch.zeros(local, dtype=torch.int32),
            "source_offsets": torch.zeros(self.num_ranks + 1, dtype=torch.int32),
            "source_expert_prefix": torch.zeros(self.num_ranks, local, dtype=torch.int32),
            "error": torch.zeros(8, dtype=torch.int32),
            "stats": torch.zeros(8, dtype=torch.int64),
            "_layout": None,
            "_expand": expand,
            "_num_tokens": x.shape[0],
            "transport_timestamps_ns": torch.zeros(2, dtype=torch.int64),
            "prefix_tx_timestamps_ns": None,
        }

    def combine(self, y: torch.Tensor, dispatch_result: Dict[str, Any], weighted: bool,
                out: Optional[torch.Tensor]) -> torch.Tensor:
        expand = bool(dispatch_result["_expand"])
        keep = {k: dispatch_result[k] for k in ("source_meta", "recv_topk_weights_full", "valid_rows")}
        if not weighted:
            keep["recv_topk_weights_full"] = torch.ones_like(keep["recv_topk_weights_full"])
        gathered = self._gather((y, keep))
        combined = reference.combine_reference(
            [g[0] for g in gathered],
            [g[1] for g in gathered],
            dispatch_result["_all_tokens"],
            do_expand=expand,
            rank=self.rank,
        )
        if out is not None:
            out.copy_(combined)
            return out
        return combined

    def pool_debug(self) -> Dict[str, Any]:
        return {"output_busy": [], "plan_busy": [], "output_sets": 0, "graph_set": False}

    def close(self) -> None:
        self._closed = True
