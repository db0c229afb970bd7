"""Memory footprint of one EP buffer: the layout arithmetic (no GPU needed) and a measurement against it.

    python benchmarks/memory_footprint.py --ranks 8 --tokens 8192                       # arithmetic only
    python benchmarks/memory_footprint.py --ranks 1 --tokens 4096 --measure             # build a buffer and measure
    python benchmarks/memory_footprint.py --ranks 1 --tokens 1024 --measure --transport host_staged

Per rank: the symmetric segment (staging rings, flags, combine area; peer-visible HBM or host memory),
the result pools (``output_pool_size`` + optional graph pool), the routing-plan pool, the combine
output pool and the combine outbox.  ``--measure`` builds a single-rank buffer and reports what the process
really took: device memory from ``cudaMemGetInfo`` before and after, host memory from ``/proc/self/smaps_rollup``
(resident and proportional set size, which is where a host-staged segment's ``/dev/shm`` pages show up).
Parity: the reference's ``benchmarks/host_buffer.py`` (independent layout arithmetic + smaps/PSS accounting; it
reports 297.3 MiB of pinned host memory per source and 2.323 GiB for 8 ranks at this shape).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def footprint(ranks: int, tokens: int, hidden: int, topk: int, experts: int, channels: int, payload_slots: int,
              pools: int, graph: bool, combine: bool, relay: bool, fused: bool = False) -> dict:
    from pcie_ep_b200 import _C

    layout = _C.segment_layout(ranks, channels, experts, topk, hidden, tokens, payload_slots, combine, fused)
    local = experts // ranks
    expanded = ranks * tokens * min(topk, local) + local * 255
    unique = ranks * tokens
    rows = max(expanded, unique)
    scalars = max(expanded, unique * topk)
    per_pool = (rows * hidden * 2 + scalars * (8 + 4) + rows * 3 * 8
                + ranks * channels * int(layout["slots_full"]) * (2 + 2 * topk) * 4)
    sets = pools + (1 if graph else 0)
    plan = tokens * 4 + tokens * ranks * 4 + tokens * topk * 4 + (ranks + experts + channels * ranks) * 4
    segment = int(layout["size_bytes"])
    result = {
        "segment_bytes": segment,
        "segment_staging_bytes": ranks * channels * int(layout["slots"]) * int(layout["row_stride"]),
        "segment_combine_bytes": ranks * tokens * int(layout["crow_stride"]) if combine else 0,
        "segment_fused_landing_bytes": tokens * topk * int(layout["crow_stride"]) if fused else 0,
        "outboxes_bytes": segment * (ranks - 1) if relay else 0,
        "result_pools_bytes": per_pool * sets,
        "plan_pool_bytes": plan * sets,
        "combine_pool_bytes": pools * tokens * hidden * 2 if combine else 0,
        # rows owned by other ranks are reduced into a local outbox before dedicated CTAs forward them
        "combine_outbox_bytes": ranks * channels * int(layout["slots_full"]) * (int(layout["crow_stride"]) + 8) if combine and ranks > 1 else 0,
        "row_stride": int(layout["row_stride"]),
        "slots": int(layout["slots"]),
        "expanded_capacity_rows": expanded,
    }
    result["total_bytes"] = (result["segment_bytes"] + result["outboxes_bytes"] + result["result_pools_bytes"]
                             + result["plan_pool_bytes"] + result["combine_pool_bytes"] + result["combine_outbox_bytes"])
    return result


def parse_smaps_rollup(text: str) -> dict:
    """``/proc/<pid>/smaps_rollup`` -> bytes per counter (Rss, Pss, Pss_Shmem, Shared_Clean, ...)."""
    counters = {}
    for line in text.splitlines():
        name, _, rest = line.partition(":")
        fields = rest.split()
        if len(fields) == 2 and fields[1] == "kB" and fields[0].isdigit():
            counters[name.strip()] = int(fields[0]) * 1024
    return counters


def host_memory() -> dict:
    try:
        return parse_smaps_rollup(Path("/proc/self/smaps_rollup").read_text())
    except OSError:
        return {}


def measure(tokens: int, hidden: int, topk: int, experts: int, channels: int, payload_slots: int, pools: int, graph: bool,
            combine: bool, transport: str) -> dict:
    """Build a one-rank buffer and report the memory it took next to what the arithmetic predicts."""
    import tempfile

    import torch
    import torch.distributed as dist

    from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer

    torch.cuda.set_device(0)
    if not dist.is_initialized():
        dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="footprint-store-"), 1), rank=0, world_size=1)
    torch.zeros(1, device="cuda")  # context and allocator pools exist before the first reading
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    host_before = host_memory()
    config = HostStagedConfig(channels=channels, payload_slots=payload_slots, descriptor_slots=payload_slots, output_pool_size=pools,
                              enable_graph=graph, enable_combine=combine, transport=transport, timeout_ms=5000)
    buffer = HostStagedEPBuffer(None, tokens, hidden, topk, experts, config)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    host_after = host_memory()
    predicted = footprint(1, tokens, hidden, topk, experts, channels, payload_slots, pools, graph, combine, False)
    buffer.close()
    host_delta = {k: host_after.get(k, 0) - host_before.get(k, 0) for k in ("Rss", "Pss", "Pss_Shmem") if k in host_after}
    device_predicted = predicted["total_bytes"] - (predicted["segment_bytes"] if transport == "host_staged" else 0)
    return {"transport": transport, "device_bytes_measured": free_before - free_after, "device_bytes_predicted": device_predicted,
            "host_bytes_measured": host_delta, "host_bytes_predicted": predicted["segment_bytes"] if transport == "host_staged" else 0,
            "arithmetic": predicted}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--measure", action="store_true", help="build a single-rank buffer on cuda:0 and measure it")
    parser.add_argument("--transport", default="peer", choices=["peer", "host_staged"])
    parser.add_argument("--ranks", type=int, default=8)
    parser.add_argument("--tokens", type=int, default=8192)
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--channels", type=int, default=128)
    parser.add_argument("--payload-slots", type=int, default=0)
    parser.add_argument("--pools", type=int, default=3)
    parser.add_argument("--graph", action="store_true")
    parser.add_argument("--no-combine", dest="combine", action="store_false")
    parser.add_argument("--relay", action="store_true")
    parser.add_argument("--fused", action="store_true", help="with the landing area of fused_expert_combine")
    args = parser.parse_args()
    if args.measure:
        print(json.dumps(measure(args.tokens, args.hidden, args.topk, args.experts, args.channels, args.payload_slots, args.pools,
                                 args.graph, args.combine, args.transport), indent=2))
        return
    result = footprint(args.ranks, args.tokens, args.hidden, args.topk, args.experts, args.channels, args.payload_slots,
                       args.pools, args.graph, args.combine, args.relay, args.fused)
    result["GiB"] = {k[:-6]: round(v / 2**30, 3) for k, v in result.items() if k.endswith("_bytes")}
    print(json.dumps(result, indent=2))


if __name__ == "__main__":
    main()
