"""Plain-PyTorch statement of the dispatch and combine semantics.

This module is the oracle every native kernel is tested against and the compute
engine of the CPU (gloo) transport.  It works from the *global view*: the list
of every source rank's ``(x, topk_idx, topk_weights)``; a caller that only has
its own inputs gathers the others first (see ``parallel/cpu_backend.py``).

Semantics (reference: ``tests/test_correctness.py:60-92`` enumerates the same
thing token by token; ``csrc/kernels/host_staged/advanced_layout.cuh:109-152``
and ``fused_receive.cuh:107-109`` define the row numbers):

* rank ``r`` owns experts ``[r*E/P, (r+1)*E/P)``;
* unique rows: every (source, token) with at least one expert on this rank,
  ordered by (source rank, source token);
* expanded rows: every (source, token, slot) whose expert is on this rank,
  ordered by (local expert, source rank, source token); expert ``e`` starts at
  ``expert_offsets[e]``, an exclusive prefix of counts rounded up to the
  alignment;
* ``stats[0]`` = source tokens with at least one remote destination,
  ``stats[1]`` = rows received from remote sources, ``stats[2]`` = remote
  (token, rank) deliveries sent.

Everything is vectorised so the oracle can be used at T=8192, H=7168 on a GPU.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..quantization import fp8_roundtrip_reference, quantize_fp8_reference

Inputs = Sequence[Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]]


def unique_capacity(num_ranks: int, num_max_tokens_per_rank: int) -> int:
    return num_ranks * num_max_tokens_per_rank


def expanded_capacity(num_ranks: int, num_max_tokens_per_rank: int, num_topk: int, num_experts: int) -> int:
    """Rows reserved for the expanded layout."""
    local = num_experts // num_ranks
    return num_ranks * num_max_tokens_per_rank * min(num_topk, local) + local * 255


def validate_routes(topk_idx: torch.Tensor, num_experts: int) -> bool:
    """True when every entry is -1 or a valid expert and no token repeats an expert."""
    if topk_idx.numel() == 0:
        return True
    ok = bool(((topk_idx >= -1) & (topk_idx < num_experts)).all())
    if not ok:
        return False
    ordered, _ = torch.sort(topk_idx, dim=1)
    repeated = (ordered[:, 1:] == ordered[:, :-1]) & (ordered[:, 1:] >= 0)
    return not bool(repeated.any())


def route_volume(topk_idx: torch.Tensor, rank: int, num_ranks: int, num_experts: int) -> Dict[str, int]:
    """Deduplicated traffic counters of one source rank."""
    local = num_experts // num_ranks
    tokens = topk_idx.shape[0]
    destinations = torch.zeros(tokens, num_ranks + 1, dtype=torch.bool, device=topk_idx.device)
    if topk_idx.numel():
        owners = torch.where(topk_idx >= 0, topk_idx // local, torch.full_like(topk_idx, num_ranks))
        destinations.scatter_(1, owners, True)
    destinations = destinations[:, :num_ranks]
    remote = destinations.clone()
    remote[:, rank] = False
    return {
        "remote_source_tokens": int(remote.any(dim=1).sum()),
        "remote_deliveries": int(remote.sum()),
        "local_tokens": int(destinations[:, rank].sum()),
        "total_deliveries": int(destinations.sum()),
        "remote_expert_branches": int(((topk_idx >= 0) & (topk_idx // local != rank)).sum()) if topk_idx.numel() else 0,
    }


def dispatch_reference(
    inputs: Inputs,
    rank: int,
    num_experts: int,
    num_max_tokens_per_rank: int,
    *,
    do_expand: bool,
    expert_alignment: int = 1,
    do_zero_padding: bool = False,
    wire_dtype: str = "bf16",
    out_dtype: Optional[torch.dtype] = None,
    recv_dtype: str = "bf16",
) -> Dict[str, torch.Tensor]:
    """Result of ``dispatch`` on ``rank`` given every source's inputs.

    The returned dict uses the native result's field names.  Rows outside the
    valid ranges are zero (payload, weights), ``-1`` (indices, metadata).
    ``recv_dtype="fp8_e4m3"``: every row (local ones too) is the E4M3 code of the source row, ``recv_x``
    is uint8 and ``recv_x_scales`` holds the row scales.
    """
    num_ranks = len(inputs)
    local = num_experts // num_ranks
    topk = inputs[0][1].shape[1]
    hidden = inputs[0][0].shape[1]
    device = inputs[0][0].device
    dtype = out_dtype or inputs[0][0].dtype
    have_weights = inputs[0][2] is not None
    keep_fp8 = recv_dtype == "fp8_e4m3"
    if keep_fp8:
        dtype = torch.uint8
    row_scales: List[torch.Tensor] = []

    src_rank: List[torch.Tensor] = []
    src_token: List[torch.Tensor] = []
    payload: List[torch.Tensor] = []
    routes: List[torch.Tensor] = []
    weights: List[torch.Tensor] = []
    source_counts = []
    stats = torch.zeros(8, dtype=torch.int64, device=device)
    for source, (x, idx, w) in enumerate(inputs):
        valid = idx >= 0
        owners = torch.where(valid, idx // local, torch.full_like(idx, -1))
        mine = owners == rank
        hit = mine.any(dim=1)
        if source == rank:
            remote = valid & ~mine
            stats[0] = int(remote.any(dim=1).sum())
            volume = route_volume(idx, rank, num_ranks, num_experts)
            stats[2] = volume["remote_deliveries"]
        else:
            stats[1] += int(hit.sum())
        tokens = torch.nonzero(hit, as_tuple=False).flatten()
        source_counts.append(int(tokens.numel()))
        src_rank.append(torch.full_like(tokens, source))
        src_token.append(tokens)
        rows = x[tokens]
        if keep_fp8:
            rows, scales = quantize_fp8_reference(rows) if rows.numel() else (rows.new_zeros(rows.shape, dtype=torch.uint8), rows.new_zeros(0, dtype=torch.float32))
            row_scales.append(scales.float())
        elif wire_dtype == "fp8_e4m3" and source != rank and rows.numel():
            rows = fp8_roundtrip_reference(rows)
        payload.append(rows.to(dtype))
        local_idx = torch.where(mine, idx - rank * local, torch.full_like(idx, -1))[tokens]
        routes.append(local_idx)
        w_full = w if w is not None else torch.ones(idx.shape, dtype=torch.float32, device=device)
        weights.append(torch.where(mine, w_full, torch.zeros_like(w_full))[tokens])

    u_rank = torch.cat(src_rank)
    u_token = torch.cat(src_token)
    u_payload = torch.cat(payload)
    u_routes = torch.cat(routes)
    u_weights = torch.cat(weights)
    u_scales = torch.cat(row_scales) if keep_fp8 else None
    unique_count = int(u_rank.numel())

    source_offsets = torch.zeros(num_ranks + 1, dtype=torch.int32, device=device)
    source_offsets[1:] = torch.tensor(source_counts, dtype=torch.int32, device=device).cumsum(0)

    # expanded branches in (unique row, slot) order, then stable sort by local expert
    branch_mask = u_routes >= 0
    b_row, b_slot = torch.nonzero(branch_mask, as_tuple=True)
    b_expert = u_routes[b_row, b_slot]
    order = torch.sort(b_expert, stable=True).indices
    b_row, b_slot, b_expert = b_row[order], b_slot[order], b_expert[order]
    expert_counts = torch.bincount(b_expert, minlength=local).to(torch.int32) if b_expert.numel() else torch.zeros(
        local, dtype=torch.int32, device=device
    )
    aligned = (expert_counts + expert_alignment - 1) // expert_alignment * expert_alignment
    expert_offsets = torch.zeros(local + 1, dtype=torch.int32, device=device)
    expert_offsets[1:] = aligned.cumsum(0)
    true_starts = torch.zeros(local, dtype=torch.int64, device=device)
    true_starts[1:] = expert_counts.cumsum(0)[:-1]
    within = torch.arange(b_expert.numel(), device=device) - true_starts[b_expert]
    e_rows = expert_offsets[:-1].long()[b_expert] + within

    # per-source per-expert exclusive prefix, as the receiver computes it
    se = torch.zeros(num_ranks, local, dtype=torch.int32, device=device)
    if b_expert.numel():
        se.index_put_((u_rank[b_row], b_expert), torch.ones_like(b_expert, dtype=torch.int32), accumulate=True)
    source_expert_prefix = torch.cumsum(se, 0) - se

    result: Dict[str, torch.Tensor] = {
        "unique_count": torch.tensor([unique_count], dtype=torch.int64, device=device),
        "expanded_count": torch.tensor([int(b_expert.numel())], dtype=torch.int64, device=device),
        "expert_counts": expert_counts,
        "expert_offsets": expert_offsets,
        "expert_prefix": (expert_offsets[:-1] + expert_counts).to(torch.int32),
        "source_offsets": source_offsets,
        "source_expert_prefix": source_expert_prefix.to(torch.int32),
        "error": torch.zeros(8, dtype=torch.int32, device=device),
        "stats": stats,
    }
    if do_expand:
        cap = expanded_capacity(num_ranks, num_max_tokens_per_rank, topk, num_experts)
        recv_x = torch.zeros(cap, hidden, dtype=dtype, device=device)
        recv_idx = torch.full((cap,), -1, dtype=torch.int64, device=device)
        recv_w = torch.zeros(cap, dtype=torch.float32, device=device)
        meta = torch.full((cap, 3), -1, dtype=torch.int64, device=device)
        recv_x[e_rows] = u_payload[b_row]
        recv_idx[e_rows] = b_expert
        recv_w[e_rows] = u_weights[b_row, b_slot]
        meta[e_rows, 0] = u_rank[b_row]
        meta[e_rows, 1] = u_token[b_row]
        meta[e_rows, 2] = b_slot
        valid_rows = torch.zeros(cap, dtype=torch.bool, device=device)
        valid_rows[e_rows] = True
        x_scales = torch.zeros(cap, dtype=torch.float32, device=device)
        if keep_fp8:
            x_scales[e_rows] = u_scales[b_row]
    else:
        cap = unique_capacity(num_ranks, num_max_tokens_per_rank)
        recv_x = torch.zeros(cap, hidden, dtype=dtype, device=device)
        recv_idx = torch.full((cap, topk), -1, dtype=torch.int64, device=device)
        recv_w = torch.zeros(cap, topk, dtype=torch.float32, device=device)
        meta = torch.full((cap, 3), -1, dtype=torch.int64, device=device)
        recv_x[:unique_count] = u_payload
        recv_idx[:unique_count] = u_routes
        recv_w[:unique_count] = u_weights
        meta[:unique_count, 0] = u_rank
        meta[:unique_count, 1] = u_token
        valid_rows = torch.zeros(cap, dtype=torch.bool, device=device)
        valid_rows[:unique_count] = True
        x_scales = torch.zeros(cap, dtype=torch.float32, device=device)
        if keep_fp8:
            x_scales[:unique_count] = u_scales
    result.update(
        recv_x_scales=x_scales if keep_fp8 else None,
        recv_x=recv_x,
        recv_topk_idx=recv_idx,
        recv_topk_weights=recv_w if have_weights else None,
        recv_topk_weights_full=recv_w,
        source_meta=meta,
        valid_rows=valid_rows,
    )
    return result


def compare_dispatch(actual: Dict[str, torch.Tensor], expected: Dict[str, torch.Tensor], *, do_expand: bool,
                     do_zero_padding: bool, have_weights: bool = True, check_stats: bool = True) -> List[str]:
    """List of human-readable mismatches between a native result and the oracle (empty = equal)."""
    problems: List[str] = []

    def same(name: str, a: torch.Tensor, b: torch.Tensor) -> None:
        a, b = a.detach().cpu(), b.detach().cpu()
        if a.shape != b.shape:
            problems.append(f"{name}: shape {tuple(a.shape)} != {tuple(b.shape)}")
        elif not torch.equal(a.to(b.dtype), b):
            bad = torch.nonzero((a.to(b.dtype) != b).reshape(a.shape[0], -1).any(dim=1)).flatten()[:4].tolist() if a.ndim else []
            problems.append(f"{name}: values differ (first rows {bad})")

    for name in ("unique_count", "expanded_count", "expert_counts", "expert_offsets", "expert_prefix",
                 "source_offsets", "source_expert_prefix"):
        if name in actual and actual[name] is not None:
            same(name, actual[name].reshape(-1), expected[name].reshape(-1))
    rows = expected["valid_rows"].cpu()
    if do_expand and do_zero_padding:
        # padding rows inside [0, expert_offsets[-1]) are defined as zero / -1 as well
        rows = rows.clone()
        rows[: int(expected["expert_offsets"][-1])] = True
    sel = torch.nonzero(rows).flatten()
    same("recv_x", actual["recv_x"].cpu()[sel].contiguous().view(torch.uint8), expected["recv_x"].cpu()[sel].contiguous().view(torch.uint8))
    if expected.get("recv_x_scales") is not None:
        same("recv_x_scales", actual["recv_x_scales"].cpu()[sel], expected["recv_x_scales"].cpu()[sel])
    same("recv_topk_idx", actual["recv_topk_idx"].cpu()[sel], expected["recv_topk_idx"].cpu()[sel])
    if have_weights and actual.get("recv_topk_weights") is not None:
        same("recv_topk_weights", actual["recv_topk_weights"].cpu()[sel], expected["recv_topk_weights_full"].cpu()[sel])
    same("source_meta", actual["source_meta"].cpu()[sel], expected["source_meta"].cpu()[sel])
    if check_stats and actual.get("stats") is not None:
        same("stats[:3]", actual["stats"].reshape(-1)[:3], expected["stats"][:3])
    if actual.get("error") is not None and int(actual["error"].reshape(-1)[0]) != 0:
        problems.append(f"error: {actual['error'].reshape(-1).tolist()}")
    return problems


def combine_reference(
    expert_outputs: Sequence[torch.Tensor],
    dispatch_results: Sequence[Dict[str, torch.Tensor]],
    num_tokens: Sequence[int],
    *,
    do_expand: bool,
    rank: int,
) -> torch.Tensor:
    """Combined ``[T, H]`` of source ``rank`` from every expert rank's output rows.

    ``expert_outputs[d]`` has the layout of ``dispatch_results[d]['recv_x']``.
    Each expert rank first reduces the rows of one source token with the
    dispatch-time weights in FP32 (expanded layout; the unique layout
    contributes its single row unweighted) and rounds that partial sum to the
    output dtype; the source then adds the partial sums in rank order in FP32.
    That is exactly the order of operations of the native combine kernel.
    """
    hidden = expert_outputs[0].shape[1]
    dtype = expert_outputs[0].dtype
    device = expert_outputs[0].device
    total = torch.zeros(num_tokens[rank], hidden, dtype=torch.float32, device=device)
    for d, (y, res) in enumerate(zip(expert_outputs, dispatch_results)):
        meta = res["source_meta"]
        rows = torch.nonzero(res["valid_rows"] & (meta[:, 0] == rank)).flatten()
        if rows.numel() == 0:
            continue
        tokens = meta[rows, 1]
        partial = torch.zeros(num_tokens[rank], hidden, dtype=torch.float32, device=device)
        if do_expand:
            w = res["recv_topk_weights_full"][rows].unsqueeze(1)
            # rows of one token are visited in increasing slot order, like the kernel does
            slots = meta[rows, 2]
            order = torch.sort(tokens * 64 + slots, stable=True).indices
            partial.index_add_(0, tokens[order], y[rows[order]].float() * w[order])
        else:
            partial.index_add_(0, tokens, y[rows].float())
        total += partial.to(dtype).float()
    return total.to(dtype)
