"""Dispatch / combine benchmark over T, routing profile, wire format and submission mode.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/benchmark.py --tokens 128 256 1024 4096 8192 --mode eager --profile uniform

Parity: the reference's ``benchmarks/benchmark.py`` (same measurement rules): every
latency is a CUDA-event interval on the submitting stream around one whole call, the per-iteration
maximum over ranks is taken and averaged; validation and reductions happen outside timed intervals;
the deduplication counters of every iteration-free check dispatch must equal the route volume.  Modes:
``eager`` (routes recomputed), ``cached`` (``cache_layout``), ``graph`` (``capture_dispatch`` dynamic)
and ``graph_cached``.  Bandwidth columns: ``logical_GBps = T*K*H*2 / t`` per GPU (the reference's
primary definition) and the NVLink roofline fraction ``(remote_deliveries * row_bytes / t) / link``.
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

from benchmarks.routing_fixture import DEFAULT_SEED, FROZEN_SPECS, FixtureSpec, frozen_manifest, load_fixture, make_routes
from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.ops.reference import route_volume

NVLINK_GBPS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool (900 nominal)


def gather(value):
    values = [None] * dist.get_world_size()
    dist.all_gather_object(values, value)
    return values


def routes_for(args, tokens: int, rank: int, world: int):
    """Skewed top-4 profiles at 8 ranks / 256 experts come from the committed frozen files (first T rows of every
    rank's table, verified against the manifest's hashes); everything else from the seeded generator."""
    spec = FixtureSpec(args.profile, tokens, args.experts, args.topk, world, args.seed)
    for frozen in FROZEN_SPECS:
        if (frozen.profile, frozen.experts, frozen.topk, frozen.world, frozen.seed) == (args.profile, args.experts, args.topk, world, args.seed) \
                and tokens <= frozen.tokens:
            _, routes = load_fixture(frozen_manifest(args.profile), tokens=tokens)
            return routes[rank], "frozen file " + frozen_manifest(args.profile).name
    return make_routes(spec, rank), "seeded generator"


def bench_one(args, tokens: int, rank: int, world: int, device: torch.device):
    wire_fp8 = args.wire == "fp8_e4m3"
    overrides = dict(channels=args.channels) if args.channels else {}
    config = HostStagedConfig.tuned(world, tokens, stage=7 if wire_fp8 else 6, wire_dtype=args.wire,
                                    enable_graph=args.mode.startswith("graph"), timeout_ms=20000, output_pool_size=2,
                                    copy_engine=args.engine, **overrides)
    (idx_cpu, w_cpu), route_source = routes_for(args, tokens, rank, world)
    volume = route_volume(idx_cpu, rank, world, args.experts)
    g = torch.Generator().manual_seed(4321 + rank)
    xs = [torch.randn(tokens, args.hidden, generator=g).to(torch.bfloat16) for _ in range(4)]
    if args.outliers:
        # one element in a hundred fifty times larger: the FP8 wire's per-token scale has to absorb it
        for x in xs:
            spikes = torch.rand(x.shape, generator=g) < 0.01
            x[spikes] *= 50
    xs = [x.to(device) for x in xs]
    idx, w = idx_cpu.to(device), w_cpu.to(device)
    record = {"tokens": tokens, "mode": args.mode, "profile": args.profile, "wire": args.wire, "topk": args.topk,
              "channels": config.channels, "world": world, "routes": route_source, "route_volume": gather(volume)}
    with HostStagedEPBuffer(dist.group.WORLD, tokens, args.hidden, args.topk, args.experts, config) as buffer:
        # one checked dispatch: counters must equal the route volume (sender / receiver dedup)
        first = buffer.dispatch(xs[0], idx, w, do_expand=True)
        buffer.check_errors()
        stats = first[3].stats.cpu().tolist()
        problems = []
        if stats[0] != volume["remote_source_tokens"] or stats[2] != volume["remote_deliveries"]:
            problems.append(f"rank {rank}: dedup counters {stats[:3]} != route volume {volume}")
        failures = [p for ps in gather(problems) for p in ps]
        if failures:
            raise AssertionError("; ".join(failures))
        cache = buffer.cache_layout(first[3]) if "cached" in args.mode else None
        del first
        graph = None
        if args.mode == "graph":
            graph = buffer.capture_dispatch(xs[0], idx, w, do_expand=True)
        elif args.mode == "graph_cached":
            graph = buffer.capture_dispatch(xs[0], topk_weights=w, handle=cache, do_expand=True)

        def dispatch(i):
            if graph is not None:
                return graph.replay()
            if cache is not None:
                return buffer.dispatch(xs[i % 4], topk_weights=w, handle=cache, do_expand=True)
            return buffer.dispatch(xs[i % 4], idx, w, do_expand=True)

        for i in range(args.warmup):
            res = dispatch(i)
            out = buffer.combine(res[0], res[3]) if args.combine else None
            del res, out
        torch.cuda.synchronize()
        dispatch_us, combine_us = [], []
        for round_index in range(args.rounds):
            dist.barrier()
            for i in range(args.iterations):
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record()
                res = dispatch(i)
                e1.record()
                out = buffer.combine(res[0], res[3]) if args.combine else None
                e2.record()
                e2.synchronize()
                dispatch_us.append(e0.elapsed_time(e1) * 1e3)
                combine_us.append(e1.elapsed_time(e2) * 1e3)
                del res, out
        buffer.check_errors()
        if graph is not None:
            graph.close()
    # per-iteration maximum over ranks, then the mean of the maxima
    all_d, all_c = gather(dispatch_us), gather(combine_us)
    max_d = [max(r[i] for r in all_d) for i in range(len(dispatch_us))]
    max_c = [max(r[i] for r in all_c) for i in range(len(combine_us))]
    row_bytes = args.hidden * (1 if wire_fp8 else 2)
    mean_d = statistics.mean(max_d)
    remote = max(v["remote_deliveries"] for v in record["route_volume"])
    record.update(
        dispatch_us_mean=mean_d, dispatch_us_p50=statistics.median(max_d), dispatch_us_min=min(max_d),
        combine_us_mean=statistics.mean(max_c) if args.combine else None,
        **bandwidth_metrics(record["route_volume"], tokens, args.topk, args.hidden, wire_fp8, mean_d),
        nvlink_roofline_us=remote * row_bytes / NVLINK_GBPS / 1e3,
        nvlink_fraction=(remote * row_bytes / NVLINK_GBPS / 1e3) / mean_d if world > 1 else None,
    )
    return record


def bandwidth_metrics(route_volumes, tokens: int, topk: int, hidden: int, wire_fp8: bool, mean_us: float) -> dict:
    """The reference's bandwidth definitions for one measured dispatch latency (decimal GB/s).

    ``logical_GBps``: ``T*K*H*2 / t`` per GPU -- every top-k branch, before deduplication, no world-size factor (the
    published comparison metric).  ``remote_delivery_GBps_total`` / ``_per_gpu``: ``F*B / t`` with F the deduplicated
    (token, destination rank) pairs that leave their rank, summed over the ranks, and B the payload bytes of a row
    (``2H`` for BF16, ``H + 4`` for the FP8 wire with its scale): what actually crossed the links, metadata and local
    rows excluded."""
    payload = hidden + 4 if wire_fp8 else hidden * 2
    deliveries = sum(v["remote_deliveries"] for v in route_volumes)
    seconds = mean_us * 1e-6
    total = deliveries * payload / seconds / 1e9
    return {"logical_GBps": tokens * topk * hidden * 2 / seconds / 1e9,
            "remote_delivery_GBps_total": total,
            "remote_delivery_GBps_per_gpu": total / max(1, len(route_volumes))}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--tokens", type=int, nargs="+", default=[128, 256, 1024, 4096, 8192])
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--mode", default="eager", choices=["eager", "cached", "graph", "graph_cached"])
    parser.add_argument("--profile", default="uniform", choices=["uniform", "hotspot_20_80", "zipf", "nvidia_calibrated"])
    parser.add_argument("--outliers", action="store_true", help="x ~ N(0,1) with 1%% of the elements multiplied by 50")
    parser.add_argument("--wire", default="bf16", choices=["bf16", "fp8_e4m3"])
    parser.add_argument("--engine", default="tma", choices=["tma", "vector"])
    parser.add_argument("--channels", type=int, default=0)
    parser.add_argument("--seed", type=int, default=DEFAULT_SEED)
    parser.add_argument("--rounds", type=int, default=2)
    parser.add_argument("--iterations", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--no-combine", dest="combine", action="store_false")
    parser.add_argument("--output", type=Path, default=None)
    args = parser.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_PORT=os.environ.get("MASTER_PORT", "29555"))
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    records = [bench_one(args, tokens, rank, world, device) for tokens in args.tokens]
    if rank == 0:
        print(f"{'T':>6} {'dispatch us':>12} {'combine us':>11} {'logical GB/s':>13} {'NVLink frac':>12}")
        for r in records:
            frac = f"{r['nvlink_fraction']:.2f}" if r["nvlink_fraction"] is not None else "-"
            comb = f"{r['combine_us_mean']:.1f}" if r["combine_us_mean"] is not None else "-"
            print(f"{r['tokens']:>6} {r['dispatch_us_mean']:>12.1f} {comb:>11} {r['logical_GBps']:>13.1f} {frac:>12}")
        if args.output:
            args.output.parent.mkdir(parents=True, exist_ok=True)
            from pcie_ep_b200 import _C

            args.output.write_text(json.dumps({"arguments": {k: str(v) for k, v in vars(args).items()},
                                               "source_fingerprint": _C.source_fingerprint()[:16], "records": records}, indent=2))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
