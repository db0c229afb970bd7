"""Small, self-terminating single-GPU workload for profilers (ncu, torch profiler).

    python benchmarks/profile_dispatch.py --tokens 2048 --iterations 3 --what all
    ncu --set full --clock-control none -k regex:dispatch_kernel -s 2 -c 1 -o prof python benchmarks/profile_dispatch.py ...

One rank (world size 1): the kernels never wait for another process, so a profiler may replay them.
Each iteration is dispatch -> grouped SwiGLU FFN -> combine at the headline shape (hidden 7168,
256 experts, top-8); NVTX ranges mark the three stages (parity: the reference's profiling driver,
benchmarks/profile_dispatch.py, NVTX + record_function markers).
"""

from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch
import torch.distributed as dist

from benchmarks.routing_fixture import DEFAULT_SEED, FixtureSpec, make_routes
from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.models.moe_layer import MoELayer
from pcie_ep_b200.ops.grouped_ffn import grouped_gemm


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--intermediate", type=int, default=2048)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--iterations", type=int, default=3)
    parser.add_argument("--channels", type=int, default=128)
    parser.add_argument("--what", default="all", choices=["all", "exchange", "gemm"])
    parser.add_argument("--wire", default="bf16", choices=["bf16", "fp8_e4m3"])
    args = parser.parse_args()
    torch.cuda.set_device(0)
    dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="profile-store-"), 1), rank=0, world_size=1)
    config = HostStagedConfig.tuned(1, args.tokens, channels=args.channels, timeout_ms=20000, output_pool_size=2,
                                    stage=7, wire_dtype=args.wire)
    idx, w = make_routes(FixtureSpec("uniform", args.tokens, args.experts, args.topk, 1, DEFAULT_SEED), 0)
    idx, w = idx.cuda(), w.cuda()
    x = torch.randn(args.tokens, args.hidden, device="cuda").to(torch.bfloat16)
    with HostStagedEPBuffer(None, args.tokens, args.hidden, args.topk, args.experts, config) as buffer:
        layer = MoELayer(buffer, args.intermediate, seed=1, with_router=False) if args.what != "exchange" else None
        for _ in range(args.iterations):
            torch.cuda.nvtx.range_push("dispatch")
            recv_x, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=True)
            torch.cuda.nvtx.range_pop()
            rows = recv_x
            if layer is not None:
                torch.cuda.nvtx.range_push("expert_ffn")
                hidden_rows, out_rows = layer._buffers(recv_x.shape[0])
                grouped_gemm(recv_x, layer.w_gate_up, handle.expert_offsets, handle.expert_counts, swiglu=True,
                             out=hidden_rows, status=layer.gemm_status)
                grouped_gemm(hidden_rows, layer.w_down, handle.expert_offsets, handle.expert_counts, swiglu=False,
                             out=out_rows, status=layer.gemm_status)
                torch.cuda.nvtx.range_pop()
                rows = out_rows
            if args.what != "gemm":
                torch.cuda.nvtx.range_push("combine")
                out, _, _ = buffer.combine(rows, handle)
                torch.cuda.nvtx.range_pop()
                del out
            del recv_x, handle
        torch.cuda.synchronize()
        buffer.check_errors()
    dist.destroy_process_group()
    print("profile workload done")


if __name__ == "__main__":
    main()
