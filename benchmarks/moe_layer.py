"""Full MoE layer round trip (BASELINE config 5): dispatch -> grouped SwiGLU expert FFN (tcgen05) ->
weighted combine, T tokens per rank, hidden 7168, 256 experts top-8, intermediate 2048, random-init
BF16 weights N(0, 0.02).  Reports the step time (device, max over ranks), the split between the three
stages and the achieved expert-FFN throughput against the measured cuBLAS BF16 peak.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/moe_layer.py --tokens 4096
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch
import torch.distributed as dist

from benchmarks.routing_fixture import DEFAULT_SEED, FixtureSpec, make_routes
from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.models.moe_layer import MoELayer
from pcie_ep_b200.ops.grouped_ffn import grouped_gemm


def gather(value):
    values = [None] * dist.get_world_size()
    dist.all_gather_object(values, value)
    return values


def run_variant(args, fp8, fused, weights, x, idx, w, rank, world, peak) -> None:
    config = HostStagedConfig.tuned(world, args.tokens, timeout_ms=20000, output_pool_size=2, stage=7 if fp8 else 6,
                                    wire_dtype="fp8_e4m3" if fp8 else "bf16", recv_dtype="fp8_e4m3" if fp8 else "bf16",
                                    fused_expert_combine=fused)
    with HostStagedEPBuffer(dist.group.WORLD, args.tokens, args.hidden, args.topk, args.experts, config) as buffer:
        layer = MoELayer(buffer, args.intermediate, seed=1, with_router=False, weights=weights)
        for _ in range(args.warmup):
            y = layer(x, idx, w)
            del y
        layer.check_errors()
        total, stage = [], []
        for _ in range(args.iterations):
            dist.barrier()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record()
            recv_x, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=True)
            e[1].record()
            hidden_rows, out_rows = layer._buffers(recv_x.shape[0])
            if layer.fp8:
                grouped_gemm(recv_x, layer.w_gate_up_fp8, handle.expert_offsets, handle.expert_counts, swiglu=True,
                             out=hidden_rows, status=layer.gemm_status, a_scales=handle._result["recv_x_scales"],
                             w_scales=layer.w_gate_up_scales)
            else:
                grouped_gemm(recv_x, layer.w_gate_up, handle.expert_offsets, handle.expert_counts, swiglu=True,
                             out=hidden_rows, status=layer.gemm_status)
            if fused:
                e[2].record()  # stage 2 = gate/up GEMM only; stage 3 = down projection + combine in one pass
                y, _, _ = buffer.fused_expert_combine(hidden_rows, layer.w_down, handle)
            else:
                grouped_gemm(hidden_rows, layer.w_down, handle.expert_offsets, handle.expert_counts, swiglu=False,
                             out=out_rows, status=layer.gemm_status)
                e[2].record()
                y, _, _ = buffer.combine(out_rows, handle)
            e[3].record()
            e[3].synchronize()
            rows = int(handle.expanded_count.item())
            stage.append([e[i].elapsed_time(e[i + 1]) * 1e3 for i in range(3)] + [rows])
            total.append(e[0].elapsed_time(e[3]) * 1e3)
            del recv_x, handle, y
        layer.check_errors()
    everyone_total = gather(total)
    everyone_stage = gather(stage)
    if rank == 0:
        per_step = [max(r[i] for r in everyone_total) for i in range(args.iterations)]
        step = statistics.median(per_step)  # median: one straggling iteration must not move the figure
        parts = [statistics.median(max(r[i][k] for r in everyone_stage) for i in range(args.iterations)) for k in range(3)]
        rows = max(r[0][3] for r in everyone_stage)
        flops = 2.0 * rows * args.hidden * args.intermediate * (2 if fused else 3)
        tflops = flops / (parts[1] * 1e-6) / 1e12
        print(json.dumps({
            "metric": "MoE layer step us (dispatch + grouped SwiGLU FFN + combine), device, max over ranks",
            "value": round(step, 1), "statistic": "median over iterations of the max over ranks",
            "slowest_iteration_us": round(max(per_step), 1), "n_gpus": world, "fp8_path": bool(fp8), "fused_down_combine": bool(fused),
            "tokens_per_rank": args.tokens, "dispatch_us": round(parts[0], 1),
            ("gate_up_gemm_us" if fused else "expert_ffn_us"): round(parts[1], 1),
            ("down_projection_plus_combine_us" if fused else "combine_us"): round(parts[2], 1),
            "expanded_rows_max": rows, "expert_ffn_tflops": round(tflops, 1),
            "fraction_of_measured_bf16_peak": round(tflops / peak, 3), "peak_tflops_used": peak,
        }), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--tokens", type=int, default=4096)
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--intermediate", type=int, default=2048)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--iterations", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--fp8", action="store_true", help="FP8 wire kept at the receiver + kind::f8f6f4 gate/up GEMM")
    parser.add_argument("--fused", action="store_true",
                        help="down projection fused with the combine send (GEMM epilogue stores into the owners' memory)")
    parser.add_argument("--variants", default="",
                        help="comma list out of bf16, fused, fp8, fp8_fused: run several variants in one process on one set "
                             "of weights (one JSON line each); overrides --fp8 / --fused")
    parser.add_argument("--peak-tflops", type=float, default=0.0, help="cuBLAS BF16 peak to report against (0: read MEASURED_PEAKS.json)")
    args = parser.parse_args()

    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_PORT=os.environ.get("MASTER_PORT", "29557"),
                          MASTER_ADDR=os.environ.get("MASTER_ADDR", "127.0.0.1"))
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    peak = args.peak_tflops
    if not peak:
        try:
            peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops_sustained"])
        except Exception:  # noqa: BLE001
            peak = 1403.0
    variants = [v for v in args.variants.split(",") if v] or [("fp8" if args.fp8 else "bf16") + ("_fused" if args.fused else "")]
    variants = ["fused" if v == "bf16_fused" else v for v in variants]
    spec = FixtureSpec("uniform", args.tokens, args.experts, args.topk, world, DEFAULT_SEED)
    idx_cpu, w_cpu = make_routes(spec, rank)
    idx, w = idx_cpu.to(device), w_cpu.to(device)
    g = torch.Generator().manual_seed(77 + rank)
    x = torch.randn(args.tokens, args.hidden, generator=g).to(torch.bfloat16).to(device)
    # random-init weights N(0, 0.02), drawn once on the device and shared by every variant
    local = args.experts // world
    wgen = torch.Generator(device=device).manual_seed(1000 + rank)
    weights = ((torch.randn(local, 2 * args.intermediate, args.hidden, device=device, generator=wgen, dtype=torch.bfloat16) * 0.02),
               (torch.randn(local, args.hidden, args.intermediate, device=device, generator=wgen, dtype=torch.bfloat16) * 0.02))
    for variant in variants:
        if variant not in ("bf16", "fused", "fp8", "fp8_fused"):
            raise SystemExit(f"unknown variant {variant}")
        run_variant(args, variant.startswith("fp8"), variant.endswith("fused"), weights, x, idx, w, rank, world, peak)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
