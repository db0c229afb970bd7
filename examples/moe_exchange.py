"""A complete expert-parallel exchange in forty lines: route, dispatch, run the local experts, combine.

    python examples/moe_exchange.py                                                                       # one rank
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/moe_exchange.py
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/moe_exchange.py --tokens 4096 --hidden 7168

One process per GPU; without GPUs the same script runs on the CPU transport (PyTorch over gloo).  Every expert here
multiplies its rows by ``1 + expert id / 100``, so the expected output of a token is known in closed form and the script
checks it: ``out[t] = sum_k w[t, k] * (1 + e[t, k] / 100) * x[t]``.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer  # noqa: E402


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--tokens", type=int, default=64)
    parser.add_argument("--hidden", type=int, default=256)
    parser.add_argument("--experts", type=int, default=16)
    parser.add_argument("--topk", type=int, default=4)
    args = parser.parse_args()

    if "RANK" in os.environ:
        dist.init_process_group("gloo")                     # control plane only: the data plane never uses it on GPUs
    else:                                                   # started without a launcher: one rank
        dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="moe-exchange-"), 1), rank=0, world_size=1)
    rank, world = dist.get_rank(), dist.get_world_size()
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    device = torch.device("cuda") if on_gpu else torch.device("cpu")
    local = args.experts // world

    g = torch.Generator().manual_seed(1 + rank)
    x = torch.randn(args.tokens, args.hidden, generator=g).to(torch.bfloat16).to(device)
    scores = torch.rand(args.tokens, args.experts, generator=g)
    weights, topk_idx = scores.topk(args.topk, dim=1)       # distinct experts per token
    weights = (weights / weights.sum(dim=1, keepdim=True)).to(device)
    topk_idx = topk_idx.to(torch.int64).to(device)

    config = HostStagedConfig.tuned(world, args.tokens) if on_gpu else HostStagedConfig(transport="cpu")
    with HostStagedEPBuffer(dist.group.WORLD, args.tokens, args.hidden, args.topk, args.experts, config) as buffer:
        recv_x, recv_expert, _, handle, _ = buffer.dispatch(x, topk_idx, weights, do_expand=True)
        # rows arrive grouped by local expert: expert e owns rows [expert_offsets[e], expert_offsets[e] + expert_counts[e])
        y = torch.zeros_like(recv_x)
        offsets, counts = handle.expert_offsets.tolist(), handle.expert_counts.tolist()
        for e in range(local):
            rows = slice(offsets[e], offsets[e] + counts[e])
            y[rows] = (recv_x[rows].float() * (1.0 + (rank * local + e) / 100.0)).to(torch.bfloat16)
        out, _, _ = buffer.combine(y, handle)               # [tokens, hidden], weighted with the dispatch-time weights
        buffer.check_errors()

    expected = ((weights * (1.0 + topk_idx.float() / 100.0)).sum(dim=1, keepdim=True) * x.float())
    error = (out.float() - expected).abs().max().item()
    worst = [None] * world
    dist.all_gather_object(worst, error)
    if rank == 0:
        print(f"{world} ranks on {'GPU' if on_gpu else 'CPU'}: {args.tokens} tokens x {args.hidden}, top-{args.topk} of {args.experts} experts; "
              f"largest deviation from the closed form {max(worst):.4f}")
    dist.destroy_process_group()
    return 0 if max(worst) < 0.1 else 1


if __name__ == "__main__":
    raise SystemExit(main())
