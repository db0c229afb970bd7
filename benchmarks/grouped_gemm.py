"""Grouped expert GEMM on one GPU at the shape one rank of an 8-way EP layer sees (32 local experts,
about T*topk/.. rows each): gate/up SwiGLU GEMM and down projection timed separately, against the
same work done as one library matmul per expert (cuBLAS through torch.mm) and against the measured
cuBLAS BF16 peak.

    python benchmarks/grouped_gemm.py --experts 32 --rows-per-expert 1024
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch

from pcie_ep_b200.ops.grouped_ffn import grouped_gemm, quantize_weights_fp8


def timed(fn, iterations: int, warmup: int, flush: torch.Tensor) -> float:
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(iterations):
        flush.zero_()  # larger than L2: every timed call starts cold
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        samples.append(start.elapsed_time(stop) * 1e3)
    return statistics.median(samples)


def scatter_timings(args, w2, flush) -> dict:
    """One emulated rank that owns every expert: T = experts * rows / topk tokens, top-8 over the local experts, so
    the expanded layout has the benchmark's shape.  Times the two-step path (plain down GEMM, combine kernel) and
    the fused one (scatter GEMM, K-slot reduction) on the same dispatch result."""
    from pcie_ep_b200 import HostStagedConfig
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    topk = 8
    tokens = args.experts * args.rows_per_expert // topk
    config = HostStagedConfig(channels=128, timeout_ms=20000, output_pool_size=2, fused_expert_combine=True)
    out = {}
    with VirtualEPGroup(1, tokens, args.hidden, topk, args.experts, config) as group:
        gen = torch.Generator(device="cuda").manual_seed(1)
        x = torch.randn(tokens, args.hidden, device="cuda", generator=gen).to(torch.bfloat16)
        idx = torch.rand(tokens, args.experts, device="cuda", generator=gen).topk(topk, dim=1).indices.contiguous()
        w = torch.softmax(torch.randn(tokens, topk, device="cuda", generator=gen), dim=1).contiguous()
        results = group.dispatch([x], [idx], [w], do_expand=True)
        rows = results[0]["recv_x"].shape[0]
        hid = (torch.randn(rows, args.intermediate, device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
        y = torch.empty(rows, args.hidden, dtype=torch.bfloat16, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        runtime = group.runtimes[0]
        offsets, counts = results[0]["expert_offsets"], results[0]["expert_counts"]
        flops = 2.0 * tokens * topk * args.hidden * args.intermediate
        t_plain = timed(lambda: grouped_gemm(hid, w2, offsets, counts, swiglu=False, out=y, status=status), args.iterations, args.warmup, flush)
        t_combine = timed(lambda: group.combine([y], results, weighted=True), args.iterations, args.warmup, flush)

        def fused_pair():
            runtime.fused_scatter_gemm(hid, w2, results[0], 0)
            runtime.fused_reduce(results[0], None, 0)

        t_fused = timed(fused_pair, args.iterations, args.warmup, flush)
        # the reduction alone: the scatter GEMM outside the timed region
        samples = []
        for _ in range(args.iterations):
            runtime.fused_scatter_gemm(hid, w2, results[0], 0)
            flush.zero_()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runtime.fused_reduce(results[0], None, 0)
            stop.record()
            stop.synchronize()
            samples.append(start.elapsed_time(stop) * 1e3)
        t_reduce = statistics.median(samples)
        assert int(runtime.fused_status()[0]) == 0 and status.tolist()[0] == 0
        out = {"scatter_case": {"tokens": tokens, "topk": topk, "rows": tokens * topk},
               "down_plain_us": round(t_plain, 1), "combine_kernel_us": round(t_combine, 1),
               "two_step_us": round(t_plain + t_combine, 1),
               "down_scatter_plus_reduce_us": round(t_fused, 1), "reduce_only_us": round(t_reduce, 1),
               "down_scatter_tflops": round(flops / max(t_fused - t_reduce, 1e-3) / 1e6, 1)}
        del results
    return out


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--experts", type=int, default=32)
    parser.add_argument("--rows-per-expert", type=int, default=1024)
    parser.add_argument("--jitter", type=float, default=0.1, help="relative spread of the expert sizes")
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--intermediate", type=int, default=2048)
    parser.add_argument("--iterations", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--fp8", action="store_true")
    parser.add_argument("--no-library", action="store_true", help="skip the per-expert torch.mm comparison")
    parser.add_argument("--scatter", action="store_true",
                        help="also time the down projection with the scatter epilogue (fused combine send) and the owner-side "
                             "reduction, on a one-rank buffer whose tokens all route to local experts")
    args = parser.parse_args()

    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(0)
    spread = (torch.rand(args.experts, generator=gen) * 2 - 1) * args.jitter
    counts = (args.rows_per_expert * (1 + spread)).round().to(torch.int32).clamp_(min=0)
    offsets = torch.zeros(args.experts + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    rows = int(offsets[-1])
    H, I, E = args.hidden, args.intermediate, args.experts
    x = (torch.randn(rows, H, device="cuda") * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16)
    hid = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    d_off, d_cnt = offsets.cuda(), counts.cuda()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    kwargs = {}
    a13, b13 = x, w13
    if args.fp8:
        amax = x.float().abs().amax(dim=1).clamp_(min=1e-8)
        scales = (amax / 448.0).contiguous()
        a13 = (x.float() / scales.unsqueeze(1)).to(torch.float8_e4m3fn)
        codes, w_scales = quantize_weights_fp8(w13.float().cpu())
        b13 = codes.cuda()
        kwargs = {"a_scales": scales, "w_scales": w_scales.cuda()}

    t_up = timed(lambda: grouped_gemm(a13, b13, d_off, d_cnt, swiglu=True, out=hid, status=status, **kwargs), args.iterations, args.warmup, flush)
    t_down = timed(lambda: grouped_gemm(hid, w2, d_off, d_cnt, swiglu=False, out=out, status=status), args.iterations, args.warmup, flush)
    assert status.tolist()[0] == 0, "a bounded wait expired"
    f_up, f_down = 2.0 * rows * H * 2 * I, 2.0 * rows * I * H
    report = {
        "rows": rows, "experts": E, "hidden": H, "intermediate": I, "fp8_gate_up": args.fp8,
        "gate_up_us": round(t_up, 1), "gate_up_tflops": round(f_up / t_up / 1e6, 1),
        "down_us": round(t_down, 1), "down_tflops": round(f_down / t_down / 1e6, 1),
        "ffn_tflops": round((f_up + f_down) / (t_up + t_down) / 1e6, 1),
    }
    if not args.no_library:
        bounds = offsets.tolist()
        full = torch.empty(rows, 2 * I, dtype=torch.bfloat16, device="cuda")

        def library_up():
            for e in range(E):
                torch.mm(x[bounds[e]:bounds[e + 1]], w13[e].t(), out=full[bounds[e]:bounds[e + 1]])

        def library_down():
            for e in range(E):
                torch.mm(hid[bounds[e]:bounds[e + 1]], w2[e].t(), out=out[bounds[e]:bounds[e + 1]])

        l_up = timed(library_up, args.iterations, args.warmup, flush)
        l_down = timed(library_down, args.iterations, args.warmup, flush)
        report.update({"library_gate_up_us_without_swiglu": round(l_up, 1), "library_gate_up_tflops": round(f_up / l_up / 1e6, 1),
                       "library_down_us": round(l_down, 1), "library_down_tflops": round(f_down / l_down / 1e6, 1)})
    if args.scatter:
        report.update(scatter_timings(args, w2, flush))
    peaks = ROOT / "MEASURED_PEAKS.json"
    if peaks.exists():
        measured = json.loads(peaks.read_text())
        report["measured_cublas_bf16_tflops"] = {k: measured[k] for k in ("bf16_tflops", "bf16_tflops_sustained") if k in measured}
    print(json.dumps(report))


if __name__ == "__main__":
    main()
