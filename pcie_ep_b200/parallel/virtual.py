"""Several EP ranks inside one process on one GPU.

Kernels of different ranks wait on one another, so they may only run as separate launches when each
launch has a GPU of its own.  With fewer GPUs than ranks the ranks are emulated as *one* cooperative
launch whose grid is (channels, ranks): every CTA of every rank is resident at once, and "peer
memory" is simply another range of the same GPU's memory.  The kernels, the protocol and the segment
layout are exactly those of the multi-GPU case; only the launch differs.

Used by the GPU tests and for single-GPU development.  Not a production path.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch

from ..config import HostStagedConfig


class VirtualEPGroup:
    def __init__(
        self,
        num_ranks: int,
        num_max_tokens_per_rank: int,
        hidden: int,
        num_topk: int,
        num_experts: int,
        config: Optional[HostStagedConfig] = None,
        device: Optional[int] = None,
    ) -> None:
        from .. import _C

        self._C = _C
        self.config = config or HostStagedConfig()
        self.num_ranks = num_ranks
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.hidden, self.num_topk, self.num_experts = hidden, num_topk, num_experts
        self.device = torch.cuda.current_device() if device is None else device
        layout = _C.segment_layout(
            num_ranks, self.config.channels, num_experts, num_topk, hidden, num_max_tokens_per_rank,
            self.config.payload_slots, self.config.enable_combine, self.config.fused_expert_combine,
        )
        self.segment_bytes = int(layout["size_bytes"])
        self.layout = layout
        self.pointers: List[int] = [_C.allocate_device_segment(self.segment_bytes, self.device) for _ in range(num_ranks)]
        options = self.config.native_options()
        self.runtimes = [
            _C.Runtime(r, num_ranks, num_max_tokens_per_rank, hidden, num_topk, num_experts, options, self.pointers,
                       self.device)
            for r in range(num_ranks)
        ]
        self._closed = False

    def dispatch(
        self,
        xs: Sequence[torch.Tensor],
        idxs: Sequence[torch.Tensor],
        weights: Sequence[Optional[torch.Tensor]],
        *,
        do_expand: bool,
        expert_alignment: int = 1,
        do_zero_padding: bool = False,
        cached: Optional[Sequence[Any]] = None,
        graph_pool: bool = False,
    ) -> List[Dict[str, Any]]:
        cached_list = list(cached) if cached is not None else [None] * self.num_ranks
        return self._C.dispatch_group(
            self.runtimes, list(xs), list(idxs), list(weights), expert_alignment, do_expand, do_zero_padding,
            cached_list, graph_pool, self.device,
        )

    def combine(self, ys: Sequence[torch.Tensor], results: Sequence[Dict[str, Any]], weighted: bool = True) -> List[torch.Tensor]:
        return self._C.combine_group(self.runtimes, list(ys), list(results), weighted, self.device)

    def fused_expert_combine(self, hidden_rows: Sequence[torch.Tensor], w_down: Sequence[torch.Tensor],
                             results: Sequence[Dict[str, Any]], ranks: Optional[Sequence[int]] = None) -> List[torch.Tensor]:
        """Down projection + combine of every virtual rank: all scatter GEMMs first (launches of one stream run in
        order, and a reduction waits for every rank's GEMM), then every rank's reduction.  ``ranks`` restricts the
        GEMMs to some ranks (tests of the bounded wait: the others never signal)."""
        active = range(self.num_ranks) if ranks is None else ranks
        for r in active:
            self.runtimes[r].fused_scatter_gemm(hidden_rows[r], w_down[r], results[r], 0)
        return [self.runtimes[r].fused_reduce(results[r], None, 0) for r in active]

    def errors(self, results: Sequence[Dict[str, Any]]) -> List[List[int]]:
        torch.cuda.synchronize(self.device)
        return [r["error"].cpu().tolist() for r in results]

    def close(self) -> None:
        if self._closed:
            return
        torch.cuda.synchronize(self.device)
        for runtime in self.runtimes:
            runtime.close()
        self.runtimes = []
        for ptr in self.pointers:
            self._C.free_device_segment(ptr)
        self.pointers = []
        self._closed = True

    def __enter__(self) -> "VirtualEPGroup":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()
