"""Memory footprint of one EP buffer, computed from the layout arithmetic alone (no GPU needed).

    python benchmarks/memory_footprint.py --ranks 8 --tokens 8192

Per rank: the symmetric segment (staging rings, flags, combine area; peer-visible HBM or host memory),
the result pools (``output_pool_size`` + optional graph pool), the routing-plan pool and the combine
output pool.  Counterpart of the reference's host-buffer accounting (``benchmarks/host_buffer.py:85-124``
there: 297.3 MiB of pinned host memory per source, 2.323 GiB for 8 ranks in direct mode, 3.492 GiB in
relay mode at the same shape, ``RESULTS_HOST_BUFFER.md:19-21``).
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
        "row_stride": int(layout["row_stride"]),
        "slots": int(layout["slots"]),
        "expanded_capacity_rows": expanded,
    }
    result["total_bytes"] = (result["segment_bytes"] + result["outboxes_bytes"] + result["result_pools_bytes"]
                             + result["plan_pool_bytes"] + result["combine_pool_bytes"])
    return result


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
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
    result = footprint(args.ranks, args.tokens, args.hidden, args.topk, args.experts, args.channels, args.payload_slots,
                       args.pools, args.graph, args.combine, args.relay, args.fused)
    result["GiB"] = {k[:-6]: round(v / 2**30, 3) for k, v in result.items() if k.endswith("_bytes")}
    print(json.dumps(result, indent=2))


if __name__ == "__main__":
    main()
