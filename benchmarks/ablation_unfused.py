"""Fused receive + expand against the two-step form (receive unique rows, then a separate scatter pass).

    python benchmarks/ablation_unfused.py --tokens 1024 4096
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/ablation_unfused.py --tokens 4096

Both forms start from the same inputs on the same buffer.  The fused form is ``dispatch(..., do_expand=True)``; the
two-step form is ``dispatch(..., do_expand=False)`` followed by ``pcie_ep_b200.ops.unfused_expand.scatter_expert_inputs``
(device-side tensor operations, no read-back).  Before anything is timed the two results are compared on the GPU:
expert counts, offsets and every valid row must be equal.  Times are CUDA-event intervals around the whole call(s),
maximum over ranks per iteration, mean of the maxima (the rules of ``benchmarks/benchmark.py``).

Parity: the reference keeps its separate ``scatter_expert_inputs`` kernel for the same comparison (its non-fused
ablation); here the product path has no such kernel, the second pass exists for this measurement only.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch
import torch.distributed as dist

from benchmarks.routing_fixture import DEFAULT_SEED, FixtureSpec, make_routes
from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.ops.unfused_expand import scatter_expert_inputs


def gather(value):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, value)
    return out


def run_case(args, tokens: int, rank: int, world: int, device: torch.device) -> dict:
    config = HostStagedConfig.tuned(world, tokens, timeout_ms=20000, output_pool_size=3)
    idx_cpu, w_cpu = make_routes(FixtureSpec("uniform", tokens, args.experts, args.topk, world, DEFAULT_SEED), rank)
    g = torch.Generator().manual_seed(99 + rank)
    x = torch.randn(tokens, args.hidden, generator=g).to(torch.bfloat16).to(device)
    idx, w = idx_cpu.to(device), w_cpu.to(device)
    local = args.experts // world
    with HostStagedEPBuffer(dist.group.WORLD, tokens, args.hidden, args.topk, args.experts, config) as buffer:
        capacity = int(buffer.runtime.expanded_capacity())

        def fused():
            return buffer.dispatch(x, idx, w, do_expand=True)

        def two_step():
            recv_x, recv_idx, recv_w, handle, _ = buffer.dispatch(x, idx, w, do_expand=False)
            return scatter_expert_inputs(recv_x, recv_idx, recv_w, handle.num_recv_tokens, local, capacity), handle

        # the two forms agree, checked on the device and reduced to one flag before anything is read back
        a = fused()
        b, b_handle = two_step()
        same = (torch.equal(a[3].expert_counts.to(torch.int32), b["expert_counts"])
                and torch.equal(a[3].expert_offsets.to(torch.int32)[: local + 1], b["expert_offsets"]))
        rows = int(b["expert_offsets"][-1])
        same = same and torch.equal(a[0][:rows], b["recv_x"][:rows]) and torch.equal(a[2][:rows], b["recv_topk_weights"][:rows])
        buffer.check_errors()
        del a, b, b_handle
        if not all(gather(bool(same))):
            raise AssertionError("the two-step form and the fused kernel disagree")

        def timed(call):
            for _ in range(args.warmup):
                out = call()
                del out
            torch.cuda.synchronize()
            samples = []
            dist.barrier()
            for _ in range(args.iterations):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = call()
                e1.record()
                e1.synchronize()
                samples.append(e0.elapsed_time(e1) * 1e3)
                del out
            every = gather(samples)
            return statistics.mean(max(r[i] for r in every) for i in range(len(samples)))

        fused_us = timed(fused)
        two_step_us = timed(two_step)
        buffer.check_errors()
    return {"tokens": tokens, "world": world, "fused_dispatch_us": fused_us, "receive_then_scatter_us": two_step_us,
            "rows_compared": rows}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--tokens", type=int, nargs="+", default=[1024, 4096])
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--iterations", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    args = parser.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world == 1:
        dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="ablation-store-"), 1), rank=0, world_size=1)
    else:
        dist.init_process_group("gloo")
    device = torch.device("cuda", local_rank)
    for tokens in args.tokens:
        record = run_case(args, tokens, rank, world, device)
        if rank == 0:
            print(json.dumps(record), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
