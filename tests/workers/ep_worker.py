"""Multi-process test program: one EP rank per process, driven through the public ``EPBuffer`` API.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P tests/workers/ep_worker.py --transport cpu|peer|host_staged --suite NAME

Every rank checks its own result against the oracle (inputs are exchanged with ``all_gather_object``
over gloo), failures are gathered so that all ranks exit non-zero together -- the structure of the
reference's torchrun tests (``tests/test_correctness.py:26-29,186-226``).
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch
import torch.distributed as dist

from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.ops import reference
from tests.helpers import make_inputs


def gather(value, group=None):
    values = [None] * dist.get_world_size(group)
    dist.all_gather_object(values, value, group=group)
    return values


def agree(failure, label):
    failures = [f for f in gather(failure) if f]
    if failures:
        raise AssertionError(f"{label}: " + "; ".join(failures))


def to_device(inputs, device):
    return tuple(None if t is None else t.to(device) for t in inputs)


def run_case(buffer, args, rank, world, device, case, dims, wire="bf16"):
    experts, topk, hidden, tmax = dims
    tokens = case["tokens"]
    if case.get("unequal"):
        tokens = 0 if rank == 0 else max(1, tokens - rank * 3)
    dtype = torch.float32 if args.transport == "cpu" and args.fp32 else torch.bfloat16
    mine = make_inputs(rank, world, tokens, hidden, experts, topk, case["pattern"], seed=case.get("seed", 7), dtype=dtype,
                       weights=case.get("weights", True))
    everyone = gather(mine)
    x, idx, w = to_device(mine, device)
    failure = None
    try:
        recv_x, recv_idx, recv_w, handle, event = buffer.dispatch(
            x, topk_idx=idx, topk_weights=w, do_expand=case["expand"], expert_alignment=case["alignment"],
            do_cpu_sync=False, do_zero_padding=case["expand"])
        event.current_stream_wait()
        buffer.check_errors()
        expected = reference.dispatch_reference(everyone, rank, experts, tmax, do_expand=case["expand"],
                                                expert_alignment=case["alignment"], do_zero_padding=case["expand"],
                                                wire_dtype=wire)
        actual = dict(handle._result)
        actual["recv_topk_weights"] = recv_w
        problems = reference.compare_dispatch(actual, expected, do_expand=case["expand"], do_zero_padding=case["expand"],
                                              have_weights=case.get("weights", True))
        if (recv_w is None) != (not case.get("weights", True)):
            problems.append("recv_topk_weights presence does not follow the input")
        if case.get("combine", True) and not problems:
            # identity experts: combine(recv_x) == x * sum of the token's weights (expanded) / number of ranks hit (unique)
            combined, _, cevent = buffer.combine(recv_x, handle)
            cevent.current_stream_wait()
            buffer.check_errors()
            xs, idxs, ws = mine
            valid = idxs >= 0
            if case["expand"]:
                weights = ws if ws is not None else torch.ones(idxs.shape)
                factor = (weights * valid).sum(dim=1, keepdim=True)
            else:
                owners = torch.where(valid, idxs // (experts // world), torch.full_like(idxs, world))
                hit = torch.zeros(idxs.shape[0], world + 1, dtype=torch.bool)
                if idxs.numel():
                    hit.scatter_(1, owners, True)
                factor = hit[:, :world].sum(dim=1, keepdim=True).float()
            want = xs.float() * factor
            got = combined.detach().cpu().float()
            if got.shape != want.shape or not torch.allclose(got, want, rtol=3e-2, atol=3e-2):
                worst = (got - want).abs().max().item() if got.shape == want.shape and got.numel() else -1
                problems.append(f"combine mismatch (max abs err {worst})")
        if problems:
            failure = f"rank {rank} case {case}: {problems}"
    except Exception as exc:  # noqa: BLE001 - reported collectively
        failure = f"rank {rank} case {case}: {type(exc).__name__}: {exc}"
    agree(failure, "case failed")


def suite_correctness(args, rank, world, device):
    experts, topk, hidden, tmax = 8 * world if args.small else 32 * world // max(1, world // 8), 4, args.hidden, 48
    experts = max(experts, world * 2)
    dims = (experts, topk, hidden, tmax)
    relay = args.numa_mode == "relay"
    config = HostStagedConfig(channels=args.channels, timeout_ms=args.timeout_ms, transport=args.transport,
                              tx_warps=2, rx_warps=3, payload_slots=args.payload_slots,
                              descriptor_slots=args.payload_slots, stage=8 if relay else 6, numa_mode=args.numa_mode,
                              relay_workers_per_numa=2 if relay else 1, combine_reduce=args.combine_reduce)
    with HostStagedEPBuffer(dist.group.WORLD, tmax, hidden, topk, experts, config) as buffer:
        cases = [dict(pattern=p, tokens=17, expand=e, alignment=1)
                 for p in ["random", "local", "multicast", "hotspot", "partial", "none"] for e in (False, True)]
        cases += [dict(pattern="random", tokens=t, unequal=u, expand=True, alignment=a)
                  for t, u, a in [(0, False, 1), (48, True, 1), (33, False, 16)]]
        cases += [dict(pattern="random", tokens=3 + i % 5, expand=bool(i % 2), alignment=8, seed=100 + i) for i in range(4)]
        cases.append(dict(pattern="multicast", tokens=5, expand=True, alignment=1, weights=False))
        for case in cases:
            run_case(buffer, args, rank, world, device, case, dims)
        if relay and world > 1:
            flows = buffer.relay.diagnostics()["flows"]
            failure = None
            if len(flows) != world - 1 or any(f["failure"] for f in flows) or not any(f["rows_copied"] for f in flows):
                failure = f"rank {rank}: relay diagnostics {flows}"
            agree(failure, "relay")
    return len(cases)


def suite_oracle_config(args, rank, world, device):
    """BASELINE config 1: T=64, hidden=128, fp32, 8 experts, top-2, softmax weights, seed 0."""
    experts, topk, hidden, tmax = 8, 2, 128, 64
    config = HostStagedConfig(channels=2, transport=args.transport, timeout_ms=args.timeout_ms)
    g = torch.Generator().manual_seed(0 + rank)
    x = torch.randn(tmax, hidden, generator=g, dtype=torch.float32)
    idx = torch.rand(tmax, experts, generator=g).topk(topk, dim=1).indices.to(torch.int64)
    w = torch.softmax(torch.randn(tmax, topk, generator=g), dim=1)
    if args.transport != "cpu":
        x = x.to(torch.bfloat16)
    everyone = gather((x, idx, w))
    with HostStagedEPBuffer(dist.group.WORLD, tmax, hidden, topk, experts, config) as buffer:
        for expand in (False, True):
            xs, ids, ws = to_device((x, idx, w), device)
            recv_x, recv_idx, recv_w, handle, event = buffer.dispatch(xs, ids, ws, do_expand=expand)
            event.current_stream_wait()
            buffer.check_errors()
            expected = reference.dispatch_reference(everyone, rank, experts, tmax, do_expand=expand)
            actual = dict(handle._result)
            problems = reference.compare_dispatch(actual, expected, do_expand=expand, do_zero_padding=False)
            agree(f"rank {rank}: {problems}" if problems else None, "oracle config")
    return 2


def suite_moe_layer(args, rank, world, device):
    """Full MoE layer (router -> dispatch -> grouped SwiGLU FFN -> combine) against a dense FP32 evaluation."""
    from pcie_ep_b200.models.moe_layer import MoELayer, dense_moe_reference

    experts, topk, hidden, inter, tmax = 4 * world, 2, args.hidden, 128, 96
    fp8 = args.fp8_layer
    config = HostStagedConfig(channels=args.channels, transport=args.transport, timeout_ms=args.timeout_ms,
                              tx_warps=2, rx_warps=3, stage=7 if fp8 else 6, wire_dtype="fp8_e4m3" if fp8 else "bf16",
                              recv_dtype="fp8_e4m3" if fp8 else "bf16", fused_expert_combine=args.fused_layer,
                              combine_reduce=args.combine_reduce)
    on_gpu = args.transport != "cpu"
    with HostStagedEPBuffer(dist.group.WORLD, tmax, hidden, topk, experts, config) as buffer:
        layer = MoELayer(buffer, inter, seed=5)
        for step, tokens in enumerate([tmax, 7 + rank, tmax - rank]):
            g = torch.Generator().manual_seed(100 * step + rank)
            x = torch.randn(tokens, hidden, generator=g).to(layer.dtype)
            xd = x.to(device)
            idx, w = layer.route(xd)
            y = layer(xd, idx, w)
            layer.check_errors()
            want = dense_moe_reference(x, idx.cpu(), w.cpu(), 5, hidden, inter,
                                       weight_dtype=torch.bfloat16 if on_gpu else torch.float32, fp8=fp8)
            got = y.detach().cpu().float()
            tol = 3e-2 if on_gpu else 1e-4
            ok = got.shape == want.shape and torch.allclose(got, want, rtol=tol, atol=tol * max(1.0, float(want.abs().max())))
            worst = float((got - want).abs().max()) if got.shape == want.shape and got.numel() else 0.0
            agree(None if ok else f"rank {rank} step {step}: max abs err {worst}", "moe layer")
    return 3


def suite_litmus(args, rank, world, device):
    """Two processes, two GPUs: READY/ACK ping-pong over NVLink-mapped HBM with bounded waits."""
    from pcie_ep_b200 import _C

    assert world == 2, "the litmus has exactly two sides"
    size, rounds, words = 1 << 20, 20000, 1024
    own = _C.allocate_device_segment(size, device.index)
    handles = gather(_C.export_device_segment(own))
    peer = _C.import_device_segment(handles[1 - rank], device.index)
    # method 0: ordinary stores + st.release.sys; method 1: the send warps' chain (bulk copy, completion wait,
    # flag stored by another lane without a system-scope fence; bulk load behind fence.proxy.async on the other side)
    for method, name in ((0, "stores+release"), (1, "bulk copy, flag after completion")):
        status = torch.zeros(4, dtype=torch.int64, device=device)
        dist.barrier()
        _C.litmus(own, peer, rank, rounds, words, status, 5000, device.index, method)
        torch.cuda.synchronize()
        timed_out, mismatches, done, elapsed = status.cpu().tolist()
        failure = None
        if timed_out or mismatches or done != rounds:
            failure = f"rank {rank} method {method}: timed_out={timed_out} mismatches={mismatches} rounds={done}/{rounds}"
        agree(failure, "litmus")
        if rank == 0:
            print(f"litmus: [{name}] {rounds} rounds, {elapsed / rounds / 1000:.2f} us per READY/ACK round trip with {words * 8} payload bytes", flush=True)
    dist.barrier()
    _C.release_imported_segment(peer)
    dist.barrier()
    _C.free_device_segment(own)
    return 1


def suite_large(args, rank, world, device):
    """Payload validation at the headline shape (parity: the reference's tests/test_large.py:54-170): hidden 7168,
    256 experts, top-8, T = 4096 / 8192 tokens per rank, BF16 and FP8 wire, dispatch (expanded) + combine.

    Every token row is a hash of (source rank, token, column), so each rank regenerates on its GPU what every row
    it received must contain, from the row's own (source, token) metadata, and compares chunk by chunk; the dedup
    counters are compared with the route volume computed from all ranks' routing tables."""
    import bench
    from pcie_ep_b200.quantization import fp8_roundtrip_reference

    hidden, experts, topk = 7168, 256, 8
    local = experts // world
    elements, cases = 0, 0
    for tokens in [int(t) for t in args.tokens.split(",")]:
        for wire in ("bf16", "fp8_e4m3"):
            config = HostStagedConfig.tuned(world, tokens, transport=args.transport, timeout_ms=args.timeout_ms, output_pool_size=2,
                                            stage=7 if wire != "bf16" else 6, wire_dtype=wire)
            idx_cpu, w_cpu = bench.make_routes(tokens, experts, topk, rank)
            all_idx = gather(idx_cpu)
            x = bench.hashed_tokens(rank, tokens, hidden, device)
            idx, w = idx_cpu.to(device), w_cpu.to(device)
            failure = None
            with HostStagedEPBuffer(dist.group.WORLD, tokens, hidden, topk, experts, config) as buffer:
                try:
                    recv_x, recv_idx, recv_w, handle, _ = buffer.dispatch(x, idx, w, do_expand=True)
                    combined, _, _ = buffer.combine(recv_x, handle)
                    torch.cuda.synchronize()
                    buffer.check_errors()
                    rows = int(handle.expanded_count)
                    # rows this rank's experts must receive, and the dedup counters, from everybody's routing table
                    want_rows = sum(int(((table // local) == rank).sum()) for table in all_idx)
                    hits = idx_cpu // local
                    want_sources = int((hits != rank).any(dim=1).sum())
                    want_deliveries = sum(int((hits == d).any(dim=1).sum()) for d in range(world) if d != rank)
                    want_received = sum(int(((table // local) == rank).any(dim=1).sum()) for s, table in enumerate(all_idx) if s != rank)
                    stats = handle.stats.cpu().tolist()
                    problems = []
                    if rows != want_rows:
                        problems.append(f"expanded rows {rows} != {want_rows}")
                    if stats[:3] != [want_sources, want_received, want_deliveries]:
                        problems.append(f"dedup counters {stats[:3]} != {[want_sources, want_received, want_deliveries]}")
                    meta = handle.source_meta[:rows]
                    cols = torch.arange(hidden, device=device, dtype=torch.int64).unsqueeze(0)
                    for lo in range(0, rows, 2048):
                        part = meta[lo:lo + 2048]
                        want = (((part[:, 0:1] * 131 + part[:, 1:2] * 7 + cols * 3) % 251) - 125).to(torch.bfloat16)
                        if wire != "bf16":
                            remote = part[:, 0] != rank
                            want = torch.where(remote.unsqueeze(1), fp8_roundtrip_reference(want), want)
                        if not torch.equal(recv_x[lo:lo + part.shape[0]], want):
                            problems.append(f"payload of rows {lo}..{lo + part.shape[0]} differs from its source")
                            break
                        elements += part.shape[0] * hidden
                    tolerance = dict(rtol=3e-2, atol=1.0) if wire == "bf16" else dict(rtol=8e-2, atol=3.0)
                    if not torch.allclose(combined.float(), x.float(), **tolerance):
                        problems.append(f"combined output off by up to {float((combined.float() - x.float()).abs().max())}")
                    if problems:
                        failure = f"rank {rank} T={tokens} wire={wire}: {problems}"
                    del recv_x, recv_idx, recv_w, handle, combined
                except Exception as exc:  # noqa: BLE001 - reported collectively
                    failure = f"rank {rank} T={tokens} wire={wire}: {type(exc).__name__}: {exc}"
                agree(failure, "large payload")
            cases += 1
    total = sum(gather(elements))
    if rank == 0:
        print(f"large: {total} BF16 elements compared with their regenerated source on {world} ranks", flush=True)
    return cases


SUITES = {"large": suite_large, "litmus": suite_litmus, "correctness": suite_correctness, "oracle_config": suite_oracle_config, "moe_layer": suite_moe_layer}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--transport", default="cpu")
    parser.add_argument("--suite", default="correctness")
    parser.add_argument("--hidden", type=int, default=256)
    parser.add_argument("--channels", type=int, default=4)
    parser.add_argument("--payload-slots", type=int, default=0)
    parser.add_argument("--timeout-ms", type=int, default=5000)
    parser.add_argument("--numa-mode", default="direct")
    parser.add_argument("--fp8-layer", action="store_true")
    parser.add_argument("--fused-layer", action="store_true", help="MoE layer with the fused down-projection + combine")
    parser.add_argument("--combine-reduce", default="auto", choices=["auto", "separate", "inline"])
    parser.add_argument("--small", action="store_true")
    parser.add_argument("--fp32", action="store_true")
    parser.add_argument("--tokens", default="4096", help="suite large: tokens per rank, comma-separated")
    args = parser.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if args.transport == "cpu":
        device = torch.device("cpu")
    else:
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        torch.cuda.set_device(device)
    count = SUITES[args.suite](args, rank, world, device)
    dist.barrier()
    if rank == 0:
        print(f"OK suite={args.suite} transport={args.transport} world={world} cases={count}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
