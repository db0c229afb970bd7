"""Attribute GPU kernels to the API calls that launched them, and audit what runs inside a dispatch / combine.

    python benchmarks/analysis_dispatch_profile.py --collect trace.json --tokens 1024     # 1 GPU: record, then analyse
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
        benchmarks/analysis_dispatch_profile.py --collect trace.json --tokens 4096          # every rank runs, rank 0 records
    python benchmarks/analysis_dispatch_profile.py --trace trace.json                     # analyse a saved trace
    python benchmarks/analysis_dispatch_profile.py --roles roles.pt                       # per-role counters (instrumented build)

Parity: the reference's ``benchmarks/analysis_dispatch_profile.py`` (correlation-id attribution of kernels to
profiler markers, role-row summaries).  The input is a Chrome trace as written by ``torch.profiler``
(``export_chrome_trace``): ``user_annotation`` events are the markers (``ep.dispatch``, ``ep.combine``, ...),
``cuda_runtime`` events carry the correlation id of the launch they made, ``kernel`` / ``gpu_memcpy`` events carry the
same id.  A kernel belongs to the innermost marker that contains its *launch call* on the host timeline, wherever
the kernel itself ran.

The audit states what this transport promises: inside a marker whose name starts with ``ep.`` there is no NCCL
kernel (the payload path is this library's own kernels over peer memory), no call that synchronises the host with
the device, and no device-to-host copy.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

SYNCHRONISING_CALLS = ("cudaDeviceSynchronize", "cudaStreamSynchronize", "cudaEventSynchronize", "cuStreamSynchronize",
                       "cuCtxSynchronize", "cuEventSynchronize")
ROLE_FIELDS = ("rows", "total_ns", "load_wait_ns", "store_wait_ns", "credit_wait_ns", "prefix_wait_ns", "idle_poll_ns",
               "meta_ns", "local_rows", "quant_ns", "issue_ns", "buffer_wait_ns", "first_batch_ns", "first_issue_ns", "drain_ns")


def _events(trace: Dict[str, Any], category: str) -> List[Dict[str, Any]]:
    wanted = category.lower()
    return [e for e in trace.get("traceEvents", []) if str(e.get("cat", "")).lower() == wanted and e.get("ph") == "X"]


def _correlation(event: Dict[str, Any]) -> Optional[int]:
    args = event.get("args", {})
    for key in ("correlation", "Correlation", "External id", "correlation_id"):
        if key in args:
            return int(args[key])
    return None


def attribute(trace: Dict[str, Any]) -> Dict[str, Dict[str, Any]]:
    """marker name -> {"calls", "kernels": [(name, us)], "host_calls": [names], "device_us", "memcpy": [names]}.

    Kernels whose launch lies in no marker are collected under ``"(outside)"``.
    """
    markers = sorted(_events(trace, "user_annotation"), key=lambda e: (e["ts"], -e.get("dur", 0)))
    launches = [e for e in _events(trace, "cuda_runtime") + _events(trace, "cuda_driver")]
    device = _events(trace, "kernel") + _events(trace, "gpu_memcpy") + _events(trace, "gpu_memset")
    by_correlation: Dict[int, List[Dict[str, Any]]] = defaultdict(list)
    for e in device:
        c = _correlation(e)
        if c is not None:
            by_correlation[c].append(e)

    def innermost(ts: float, tid: Any) -> str:
        best, best_dur = "(outside)", None
        for m in markers:
            if m["ts"] <= ts <= m["ts"] + m.get("dur", 0) and (m.get("tid") == tid or tid is None or m.get("tid") is None):
                if best_dur is None or m.get("dur", 0) <= best_dur:
                    best, best_dur = m["name"], m.get("dur", 0)
        return best

    report: Dict[str, Dict[str, Any]] = defaultdict(lambda: {"calls": 0, "kernels": [], "host_calls": [], "memcpy": [], "device_us": 0.0})
    for m in markers:
        report[m["name"]]["calls"] += 1
    for call in launches:
        owner = innermost(call["ts"], call.get("tid"))
        report[owner]["host_calls"].append(call["name"])
        c = _correlation(call)
        for dev in by_correlation.get(c, []) if c is not None else []:
            entry = report[owner]
            if str(dev.get("cat", "")).lower() == "kernel":
                entry["kernels"].append((dev["name"], float(dev.get("dur", 0))))
            else:
                entry["memcpy"].append(dev["name"])
            entry["device_us"] += float(dev.get("dur", 0))
    return dict(report)


def audit(report: Dict[str, Dict[str, Any]], prefix: str = "ep.") -> List[str]:
    """Violations of the transport's promises inside markers whose name starts with ``prefix`` (empty list = clean)."""
    problems = []
    for name, entry in report.items():
        if not name.startswith(prefix):
            continue
        for kernel, _ in entry["kernels"]:
            if "nccl" in kernel.lower():
                problems.append(f"{name}: NCCL kernel {kernel} ran on the payload path")
        for call in entry["host_calls"]:
            if any(call.startswith(s) for s in SYNCHRONISING_CALLS):
                problems.append(f"{name}: host call {call} synchronises with the device")
        for copy in entry["memcpy"]:
            if "dtoh" in copy.lower().replace(" ", "").replace("-", ""):
                problems.append(f"{name}: device-to-host copy {copy}")
    return problems


def format_report(report: Dict[str, Dict[str, Any]]) -> str:
    lines = [f"{'marker':<22} {'calls':>5} {'kernels':>7} {'device us / call':>17}  kernels (mean us)"]
    for name in sorted(report):
        entry = report[name]
        calls = max(1, entry["calls"])
        per_kernel: Dict[str, List[float]] = defaultdict(list)
        for kernel, us in entry["kernels"]:
            per_kernel[kernel.split("(")[0].split("<")[0][-40:]].append(us)
        detail = ", ".join(f"{k} {statistics.mean(v):.1f}" for k, v in sorted(per_kernel.items()))
        lines.append(f"{name:<22} {entry['calls']:>5} {len(entry['kernels']):>7} {entry['device_us'] / calls:>17.1f}  {detail}")
    return "\n".join(lines)


def summarise_roles(role_profiling: Any, channels: int, send_ctas: int, tx_warps: int, rx_warps: int) -> Dict[str, Dict[str, float]]:
    """Mean per warp of every counter of the instrumented build, for the send and the receive role.

    ``role_profiling`` is the ``[CTAs, 16 warps, 16 counters]`` tensor of a dispatch result (empty in a normal build).
    With dedicated sender CTAs the send warps are warps 0.. of the CTAs behind the channel CTAs; otherwise they are
    warps 1..tx of every channel CTA and the receive warps follow them."""
    import torch

    role = torch.as_tensor(role_profiling).double()
    if role.numel() == 0:
        return {}
    if send_ctas > 0:
        send = role[channels:channels + send_ctas, :tx_warps]
        recv = role[:channels, 1:1 + rx_warps]
    else:
        send = role[:channels, 1:1 + tx_warps]
        recv = role[:channels, 1 + tx_warps:1 + tx_warps + rx_warps]
    out = {}
    for label, block in (("send", send), ("receive", recv)):
        flat = block.reshape(-1, block.shape[-1])
        out[label] = {field: float(flat[:, i].mean()) for i, field in enumerate(ROLE_FIELDS)}
        out[label]["warps"] = float(flat.shape[0])
    return out


def collect(path: Path, tokens: int, iterations: int) -> Optional[Dict[str, Any]]:
    """Record dispatch + combine under the torch profiler with ``ep.*`` markers and save rank 0's trace.

    One process: one rank on GPU 0.  Under ``torch.distributed.run`` (RANK / WORLD_SIZE / LOCAL_RANK in the environment):
    every rank runs the exchange, rank 0 records and returns the trace, the other ranks return None."""
    import os
    import tempfile

    import torch
    import torch.distributed as dist

    import bench
    from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if not dist.is_initialized():
        if world == 1:
            dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="analysis-store-"), 1), rank=0, world_size=1)
        else:
            dist.init_process_group("gloo")
    config = HostStagedConfig.tuned(world, tokens, timeout_ms=20000, output_pool_size=2)
    idx, w = bench.make_routes(tokens, 256, 8, rank)
    idx, w = idx.cuda(), w.cuda()
    x = torch.randn(tokens, 7168, device="cuda").to(torch.bfloat16)
    with HostStagedEPBuffer(None if world == 1 else dist.group.WORLD, tokens, 7168, 8, 256, config) as buffer:
        def step() -> None:
            with torch.profiler.record_function("ep.dispatch"):
                recv_x, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=True)
            with torch.profiler.record_function("ep.combine"):
                out, _, _ = buffer.combine(recv_x, handle)
            del recv_x, handle, out

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]) as prof:
            for _ in range(iterations):
                step()
            torch.cuda.synchronize()
        buffer.check_errors()
    if rank != 0:
        return None
    prof.export_chrome_trace(str(path))
    return json.loads(Path(path).read_text())


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--trace", type=Path, help="Chrome trace written by torch.profiler")
    parser.add_argument("--collect", type=Path, help="record a dispatch + combine trace to this file (rank 0's, when started with "
                        "torch.distributed.run on several GPUs), then analyse it")
    parser.add_argument("--tokens", type=int, default=1024)
    parser.add_argument("--iterations", type=int, default=5)
    parser.add_argument("--roles", type=Path, help="torch.save'd dict with role_profiling, channels, send_ctas, tx_warps, rx_warps")
    args = parser.parse_args()
    if args.roles:
        import torch

        saved = torch.load(args.roles)
        for label, fields in summarise_roles(saved["role_profiling"], saved["channels"], saved["send_ctas"], saved["tx_warps"],
                                             saved["rx_warps"]).items():
            print(label, " ".join(f"{k}={v:.1f}" for k, v in fields.items()))
    trace = None
    if args.collect:
        trace = collect(args.collect, args.tokens, args.iterations)
    elif args.trace:
        trace = json.loads(args.trace.read_text())
    if trace is not None:
        report = attribute(trace)
        print(format_report(report))
        problems = audit(report)
        print("audit:", "clean" if not problems else "; ".join(problems))
        if problems:
            raise SystemExit(1)


if __name__ == "__main__":
    main()
