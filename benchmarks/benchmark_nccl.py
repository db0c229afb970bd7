"""NCCL baselines on identical tensors: what a library-only solution costs.

``nccl_payload``   one ``all_gather_into_tensor`` of the BF16 tokens (every rank receives everything).
``nccl_dispatch``  expert-ready dispatch: pack (tokens | ids | weights) per row, one uint8 all-gather,
                   then a stable per-expert expansion of the rows this rank owns (PyTorch kernels).
``nccl_dispatch_kernels``  the same with the reference's own pack / count / prefix / scatter CUDA kernels
                   (``benchmarks/csrc/nccl_expand.cu`` of the reference, used unmodified from ``baseline/_ref`` when
                   that copy and its build exist; at most 32 experts per rank).
``fused``          this framework's fused dispatch kernel.

Parity: the reference's three-way comparison (``benchmarks/benchmark_nccl_shm.py``), which forces NCCL onto
shared memory because its target has no NVLink (``benchmarks/reference_nccl_shm.py`` runs that script as it
is); here NCCL runs over NVLink/NVSwitch as it would in production.  The expansion result is validated against
the fused kernel's output outside the timed region.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/benchmark_nccl.py --tokens 128 1024 4096
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


def gather(value):
    values = [None] * dist.get_world_size()
    dist.all_gather_object(values, value)
    return values


def pack(x, idx, w):
    return torch.cat([x.view(torch.uint8), idx.view(torch.uint8), w.view(torch.uint8)], dim=1)


def expand(rows, hidden, topk, rank, local):
    """Stable (expert, source, token) expansion of the gathered rows for this rank's experts."""
    x = rows[:, : hidden * 2].view(torch.bfloat16)
    idx = rows[:, hidden * 2: hidden * 2 + topk * 8].view(torch.int64)
    w = rows[:, hidden * 2 + topk * 8:].view(torch.float32)
    mine = (idx >= rank * local) & (idx < (rank + 1) * local)
    row, slot = torch.nonzero(mine, as_tuple=True)
    expert = idx[row, slot] - rank * local
    order = torch.sort(expert, stable=True).indices
    row, slot, expert = row[order], slot[order], expert[order]
    counts = torch.bincount(expert, minlength=local)
    return x[row], expert, w[row, slot], counts


def reference_expand(world, tokens, hidden, topk, experts, rank, device):
    """The reference's NCCLExpand helper (its pack and expansion kernels), or None when baseline/_ref has no build."""
    ref = ROOT / "baseline" / "_ref" / "benchmarks"
    if not (ref / "nccl_expand.py").exists() or experts // world > 32:
        return None
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", str(ROOT / "baseline" / "_ref_build"))
    sys.path.insert(0, str(ref))
    try:
        from nccl_expand import NCCLExpand

        return NCCLExpand(world, tokens, hidden, topk, experts, rank, device)
    except Exception as exc:  # noqa: BLE001 - the column is simply left out
        if rank == 0:
            print(f"reference expansion kernels unavailable: {type(exc).__name__}: {exc}", flush=True)
        return None


def timed(fn, iterations, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iterations):
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        samples.append(e0.elapsed_time(e1) * 1e3)
    everyone = gather(samples)
    return statistics.mean(max(r[i] for r in everyone) for i in range(iterations))


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--tokens", type=int, nargs="+", default=[128, 1024, 4096])
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--profile", default="uniform")
    parser.add_argument("--iterations", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--output", type=Path, default=None)
    args = parser.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_PORT=os.environ.get("MASTER_PORT", "29556"))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=device)
    control = dist.new_group(backend="gloo")
    local = args.experts // world
    records = []
    for tokens in args.tokens:
        spec = FixtureSpec(args.profile, tokens, args.experts, args.topk, world, DEFAULT_SEED)
        idx_cpu, w_cpu = make_routes(spec, rank)
        g = torch.Generator().manual_seed(4321 + rank)
        x = torch.randn(tokens, args.hidden, generator=g).to(torch.bfloat16).to(device)
        idx, w = idx_cpu.to(device), w_cpu.to(device)
        gathered_x = torch.empty(world * tokens, args.hidden, dtype=torch.bfloat16, device=device)
        row_bytes = args.hidden * 2 + args.topk * 12
        gathered_rows = torch.empty(world * tokens, row_bytes, dtype=torch.uint8, device=device)

        def nccl_payload():
            dist.all_gather_into_tensor(gathered_x, x)

        def nccl_dispatch():
            dist.all_gather_into_tensor(gathered_rows, pack(x, idx, w))
            return expand(gathered_rows, args.hidden, args.topk, rank, local)

        helper = reference_expand(world, tokens, args.hidden, args.topk, args.experts, rank, device)

        def nccl_dispatch_kernels():
            dist.all_gather_into_tensor(helper.packed_recv, helper.pack(x, idx, w))
            return helper.expand()

        config = HostStagedConfig.tuned(world, tokens, timeout_ms=20000, output_pool_size=2, enable_combine=False)
        buffer = HostStagedEPBuffer(dist.group.WORLD, tokens, args.hidden, args.topk, args.experts, config,
                                    control_group=control)

        def fused():
            res = buffer.dispatch(x, idx, w, do_expand=True)
            return res

        # validation outside timing: same rows per expert, same order
        rows, expert, weights, counts = nccl_dispatch()
        res = fused()
        torch.cuda.synchronize()
        handle = res[3]
        ok = torch.equal(counts.to(torch.int32), handle.expert_counts)
        offsets = handle.expert_offsets[:-1].long()
        starts = torch.cumsum(counts, 0) - counts
        position = offsets[expert] + (torch.arange(expert.numel(), device=device) - starts[expert])
        ok = ok and torch.equal(res[0][position].view(torch.int16), rows.view(torch.int16))
        ok = ok and torch.equal(res[2][position], weights)
        failures = [r for r, good in enumerate(gather(bool(ok))) if not good]
        if failures:
            raise AssertionError(f"NCCL expansion and fused dispatch disagree on ranks {failures}")
        del res, handle
        record = {
            "tokens": tokens, "world": world,
            "nccl_payload_us": timed(nccl_payload, args.iterations, args.warmup),
            "nccl_dispatch_us": timed(nccl_dispatch, args.iterations, args.warmup),
            "fused_dispatch_us": timed(lambda: fused(), args.iterations, args.warmup),
        }
        if helper is not None:
            record["nccl_dispatch_kernels_us"] = timed(nccl_dispatch_kernels, args.iterations, args.warmup)
        buffer.close()
        records.append(record)
        if rank == 0:
            print(json.dumps(record), flush=True)
    if rank == 0 and args.output:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        args.output.write_text(json.dumps(records, indent=2))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
