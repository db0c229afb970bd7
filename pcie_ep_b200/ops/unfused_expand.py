"""The separate expansion step of a non-fused dispatch -- an ablation, not the product path.

``dispatch(..., do_expand=True)`` writes every received row straight into the rows of its local experts (receive and
expand are one kernel).  The reference also keeps the older two-step form for comparison: receive unique rows, then a
second pass scatters them to the experts (its ``scatter_expert_inputs``).  ``scatter_expert_inputs`` below is that second
pass for results of ``dispatch(..., do_expand=False)``: device-side tensor operations only, shapes are capacities, nothing
is read back to the host.  Its output has exactly the layout the fused kernel produces -- rows grouped by local
expert, inside an expert in the order of the unique rows (source rank, then token), every expert's segment padded to
``expert_alignment`` -- so the two forms can be compared row by row and timed against each other
(``benchmarks/ablation_unfused.py``).

The handle of the unique dispatch stays a unique-layout handle: ``combine`` with it takes unique-layout rows.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch


def scatter_expert_inputs(recv_x: torch.Tensor, recv_topk_idx: torch.Tensor, recv_topk_weights: Optional[torch.Tensor],
                          unique_count: torch.Tensor, num_local_experts: int, capacity: int, expert_alignment: int = 1,
                          source_meta: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """Expand unique rows to expert rows.

    ``recv_x`` ``[rows, hidden]``, ``recv_topk_idx`` ``[rows, K]`` (local expert id or -1), ``recv_topk_weights``
    ``[rows, K]`` or ``None``, ``unique_count`` a one-element tensor with the number of valid rows -- all as returned by
    a unique dispatch (the count is ``handle.num_recv_tokens``).  ``capacity`` is the number of rows of the result
    (``runtime.expanded_capacity()`` of the buffer, or anything that is large enough).  Returns ``recv_x``
    ``[capacity, hidden]`` (zero outside valid rows), ``recv_topk_idx`` ``[capacity]``, ``recv_topk_weights``
    ``[capacity]``, ``source_meta`` ``[capacity, 3]`` when given, ``expert_counts`` ``[E_local]`` int32,
    ``expert_offsets`` ``[E_local + 1]`` int32 and ``expanded_count``.
    """
    if recv_x.dim() != 2 or recv_topk_idx.dim() != 2 or recv_topk_idx.shape[0] != recv_x.shape[0]:
        raise ValueError("recv_x [rows, hidden] and recv_topk_idx [rows, K] of a unique dispatch are expected")
    if num_local_experts < 1 or capacity < 1 or expert_alignment < 1:
        raise ValueError("num_local_experts, capacity and expert_alignment must be positive")
    rows, topk = recv_topk_idx.shape
    device = recv_x.device
    experts = recv_topk_idx.reshape(-1).to(torch.int64)
    row_of_pair = torch.arange(rows, device=device).repeat_interleave(topk)
    slot_of_pair = torch.arange(topk, device=device).repeat(rows)
    valid = (experts >= 0) & (experts < num_local_experts) & (row_of_pair < unique_count.reshape(-1)[0].to(torch.int64))
    # invalid pairs sort behind every expert and end up in a spare row behind the result
    key = torch.where(valid, experts, torch.full_like(experts, num_local_experts))
    order = torch.sort(key, stable=True).indices
    key_sorted = key[order]
    counts_all = torch.bincount(key, minlength=num_local_experts + 1)
    counts = counts_all[:num_local_experts]
    padded = (counts + expert_alignment - 1) // expert_alignment * expert_alignment
    offsets = torch.zeros(num_local_experts + 1, dtype=torch.int64, device=device)
    offsets[1:] = padded.cumsum(0)
    starts_sorted = torch.zeros(num_local_experts + 1, dtype=torch.int64, device=device)  # first position of a key in sorted order
    starts_sorted[1:] = counts.cumsum(0)
    position = torch.arange(experts.numel(), device=device) - starts_sorted[key_sorted]
    spare = capacity
    destination = torch.where(key_sorted < num_local_experts, offsets[key_sorted.clamp(max=num_local_experts)] + position,
                              torch.full_like(position, spare))
    destination = torch.where(destination < capacity, destination, torch.full_like(destination, spare))  # (a result that is too small drops rows)
    source_rows = row_of_pair[order]
    out_x = torch.zeros(capacity + 1, recv_x.shape[1], dtype=recv_x.dtype, device=device)
    out_x.index_copy_(0, destination, recv_x.index_select(0, source_rows))
    out_idx = torch.full((capacity + 1,), -1, dtype=torch.int64, device=device)
    out_idx.index_copy_(0, destination, key_sorted)
    out_w = torch.zeros(capacity + 1, dtype=torch.float32, device=device)
    if recv_topk_weights is not None:
        out_w.index_copy_(0, destination, recv_topk_weights.reshape(-1).to(torch.float32)[order])
    result = {
        "recv_x": out_x[:capacity],
        "recv_topk_idx": out_idx[:capacity],
        "recv_topk_weights": out_w[:capacity] if recv_topk_weights is not None else None,
        "expert_counts": counts.to(torch.int32),
        "expert_offsets": offsets.to(torch.int32),
        "expanded_count": counts.sum().reshape(1),
    }
    if source_meta is not None:
        meta = torch.full((capacity + 1, 3), -1, dtype=source_meta.dtype, device=device)
        picked = source_meta.index_select(0, source_rows).clone()
        picked[:, 2] = slot_of_pair[order].to(source_meta.dtype)
        meta.index_copy_(0, destination, picked)
        result["source_meta"] = meta[:capacity]
    return result
