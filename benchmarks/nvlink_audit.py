"""Path evidence: the dispatch's payload crosses NVLink, once per (token, destination rank).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/nvlink_audit.py --tokens 4096 --iterations 50

Every rank reads NVML's NVLink data counters of its own GPU (transmit and receive, summed over the links; read-only
queries), runs ``--iterations`` dispatches, reads the counters again and compares the difference with what the routing
says must have crossed the link: ``remote deliveries x bytes per staged row`` sent, the other ranks' deliveries to this
rank received.  A dispatch that sent a row once per remote *expert* instead of once per remote *rank* (no source
deduplication), or that fell back to staging through host memory, shows up as a ratio far from one.  The counters also
see flags, counts messages and credit words, and other users of the same GPU; the accepted band is therefore
``[0.9, 1.3]`` of the expected volume by default.

One JSON line per rank goes to rank 0's stdout; the exit status is 0 when every rank is inside the band, 1 when not,
3 when the counters cannot be read on this machine.

Parity: the reference proves the opposite for its design with ``scripts/check_path_counters.py`` (every NVLink counter
unchanged by a run: its payload goes through host memory over PCIe).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Any, Dict, Optional, Tuple

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

ALL_LINKS = 0xFFFFFFFF  # scope of a field value: the sum over the GPU's links


def read_counters(nvml: Any, handle: Any) -> Optional[Tuple[int, int]]:
    """(bytes transmitted, bytes received) over NVLink since the driver was loaded, or None where the driver does not
    report them.  NVML counts in KiB."""
    fields = [(nvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX, ALL_LINKS), (nvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX, ALL_LINKS)]
    try:
        values = nvml.nvmlDeviceGetFieldValues(handle, fields)
    except Exception:  # noqa: BLE001 - no NVLink, or a driver without these fields
        return None
    if any(v.nvmlReturn != 0 for v in values):
        return None
    return int(values[0].value.ullVal) * 1024, int(values[1].value.ullVal) * 1024


def judge(expected_bytes: int, measured_bytes: int, low: float, high: float) -> Dict[str, Any]:
    """Ratio of measured to expected traffic and whether it is inside the accepted band.  Nothing expected (a rank
    that sends or receives nothing remotely) is fine as long as next to nothing was measured."""
    if expected_bytes <= 0:
        return {"expected_bytes": 0, "measured_bytes": measured_bytes, "ratio": None, "ok": measured_bytes < (1 << 20)}
    ratio = measured_bytes / expected_bytes
    return {"expected_bytes": expected_bytes, "measured_bytes": measured_bytes, "ratio": round(ratio, 4), "ok": low <= ratio <= high}


def expected_traffic(volumes: list, rank: int, deliveries_to: list, row_bytes: int, iterations: int) -> Tuple[int, int]:
    """(bytes this rank sends, bytes it receives) in ``iterations`` dispatches: ``volumes[r]`` is the route volume of
    rank r, ``deliveries_to[r][d]`` the number of rows rank r sends to rank d."""
    sent = volumes[rank]["remote_deliveries"] * row_bytes * iterations
    received = sum(deliveries_to[r][rank] for r in range(len(volumes)) if r != rank) * row_bytes * iterations
    return sent, received


def staged_row_bytes(hidden: int, topk: int, wire: str) -> int:
    """Bytes one row puts on the link: the payload in its wire format, rounded up to 16 bytes, then the row's metadata
    (token, scale, sequence, then expert slot, ordinal and weight per top-k entry), rounded up to 16 bytes -- the same
    arithmetic as ``SegmentLayout`` in ``csrc/kernels/protocol.cuh``."""
    def up16(n: int) -> int:
        return (n + 15) // 16 * 16

    return up16(hidden * (2 if wire == "bf16" else 1)) + up16(16 + 12 * topk)


def deliveries_per_destination(topk_idx: Any, world: int, experts: int) -> list:
    """Rows one source sends to each rank: tokens with at least one expert there."""
    import torch

    local = experts // world
    owners = torch.where(topk_idx >= 0, topk_idx // local, torch.full_like(topk_idx, world))
    hit = torch.zeros(topk_idx.shape[0], world + 1, dtype=torch.bool)
    hit.scatter_(1, owners, True)
    return [int(hit[:, d].sum()) for d in range(world)]


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--tokens", type=int, default=4096)
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--iterations", type=int, default=50)
    parser.add_argument("--wire", default="bf16", choices=["bf16", "fp8_e4m3"])
    parser.add_argument("--low", type=float, default=0.9)
    parser.add_argument("--high", type=float, default=1.3)
    args = parser.parse_args()

    import torch
    import torch.distributed as dist

    from benchmarks.routing_fixture import DEFAULT_SEED, FixtureSpec, make_routes
    from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
    from pcie_ep_b200.ops.reference import route_volume

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        print("needs at least two ranks (one process per GPU): nothing crosses NVLink with one", file=sys.stderr)
        return 2
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("gloo")

    counters = None
    try:
        import pynvml as nvml

        nvml.nvmlInit()
        handle = nvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(torch.cuda.get_device_properties(device).uuid)).encode())
        counters = lambda: read_counters(nvml, handle)  # noqa: E731
    except Exception:  # noqa: BLE001 - no NVML
        counters = lambda: None  # noqa: E731

    routes = [make_routes(FixtureSpec("uniform", args.tokens, args.experts, args.topk, world, DEFAULT_SEED), r)[0] for r in range(world)]
    idx_cpu, w_cpu = make_routes(FixtureSpec("uniform", args.tokens, args.experts, args.topk, world, DEFAULT_SEED), rank)
    volumes = [route_volume(routes[r], r, world, args.experts) for r in range(world)]
    per_destination = [deliveries_per_destination(routes[r], world, args.experts) for r in range(world)]
    # a staged row: the payload in its wire format plus the row's metadata (token, sequence, expert slots, weights)
    row_bytes = staged_row_bytes(args.hidden, args.topk, args.wire)

    config = HostStagedConfig.tuned(world, args.tokens, timeout_ms=20000, output_pool_size=2, wire_dtype=args.wire,
                                    stage=7 if args.wire != "bf16" else 6, enable_combine=False)
    x = torch.randn(args.tokens, args.hidden, generator=torch.Generator().manual_seed(7 + rank)).to(torch.bfloat16).to(device)
    idx, w = idx_cpu.to(device), w_cpu.to(device)
    with HostStagedEPBuffer(dist.group.WORLD, args.tokens, args.hidden, args.topk, args.experts, config) as buffer:
        for _ in range(3):
            out = buffer.dispatch(x, idx, w, do_expand=True)
            del out
        torch.cuda.synchronize()
        dist.barrier()
        before = counters()
        dist.barrier()
        for _ in range(args.iterations):
            out = buffer.dispatch(x, idx, w, do_expand=True)
            del out
        torch.cuda.synchronize()
        buffer.check_errors()
        dist.barrier()
        after = counters()
    sent, received = expected_traffic(volumes, rank, per_destination, row_bytes, args.iterations)
    if before is None or after is None:
        record: Dict[str, Any] = {"rank": rank, "unavailable": "NVML does not report NVLink data counters here"}
    else:
        record = {"rank": rank, "iterations": args.iterations, "row_bytes": row_bytes,
                  "transmit": judge(sent, after[0] - before[0], args.low, args.high),
                  "receive": judge(received, after[1] - before[1], args.low, args.high)}
    records = [None] * world
    dist.all_gather_object(records, record)
    dist.destroy_process_group()
    if rank == 0:
        for r in records:
            print(json.dumps(r), flush=True)
    if any("unavailable" in r for r in records):
        return 3
    return 0 if all(r["transmit"]["ok"] and r["receive"]["ok"] for r in records) else 1


if __name__ == "__main__":
    raise SystemExit(main())
