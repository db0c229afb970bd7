"""Scale, stress and host-synchronisation audits.

* headline-shaped dispatch + combine at thousands of tokens per rank against the vectorised oracle
  evaluated on the GPU (reference: tests/test_large.py checks 6.25 G elements the same way);
* thousands of back-to-back epochs over tiny rings with periodic full verification
  (reference: tests/test_stress.py);
* a profiler trace proving that dispatch/combine enqueue work without any host synchronisation or
  device-to-host copy (reference: tests/test_profiler.py)."""

import tempfile

import pytest
import torch
import torch.distributed as dist

from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.ops import reference
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


def test_headline_shape_at_scale_matches_oracle(ext):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tokens = 4, 256, 8, 7168, 2048
    config = HostStagedConfig(channels=32, timeout_ms=20000, output_pool_size=2)
    with VirtualEPGroup(world, tokens, hidden, topk, experts, config) as group:
        gen = torch.Generator(device="cuda").manual_seed(3)
        xs = [torch.randn(tokens, hidden, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(world)]
        idxs = [torch.rand(tokens, experts, device="cuda", generator=gen).topk(topk, dim=1).indices.contiguous() for _ in range(world)]
        ws = [torch.softmax(torch.randn(tokens, topk, device="cuda", generator=gen), dim=1).contiguous() for _ in range(world)]
        results = group.dispatch(xs, idxs, ws, do_expand=True)
        torch.cuda.synchronize()
        inputs = list(zip(xs, idxs, ws))
        checked = 0
        for rank in range(world):
            expected = reference.dispatch_reference(inputs, rank, experts, tokens, do_expand=True)
            rows = expected["valid_rows"]
            assert torch.equal(results[rank]["expert_counts"], expected["expert_counts"])
            assert torch.equal(results[rank]["expert_offsets"], expected["expert_offsets"])
            assert torch.equal(results[rank]["recv_x"][rows].view(torch.int16), expected["recv_x"][rows].view(torch.int16))
            assert torch.equal(results[rank]["source_meta"][rows], expected["source_meta"][rows])
            assert torch.equal(results[rank]["recv_topk_weights"][rows], expected["recv_topk_weights_full"][rows])
            assert int(results[rank]["error"][0]) == 0
            checked += int(rows.sum()) * hidden
        assert checked == world * tokens * topk * hidden
        # identity experts: combine returns sum_k w_k * x = x (softmax weights)
        outs = group.combine([r["recv_x"] for r in results], results, weighted=True)
        torch.cuda.synchronize()
        for rank in range(world):
            assert torch.allclose(outs[rank].float(), xs[rank].float(), rtol=3e-2, atol=3e-2)


def test_thousands_of_epochs_over_tiny_rings(ext):
    """3000 epochs by default; ``PCIE_EP_B200_STRESS_EPOCHS=100000`` is the long acceptance run
    (``benchmarks/run_matrix.py validate --group stress``)."""
    import os

    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    epochs = max(4, int(os.environ.get("PCIE_EP_B200_STRESS_EPOCHS", "3000")))

    world, experts, topk, hidden, tmax = 4, 16, 4, 128, 24
    config = HostStagedConfig(channels=2, payload_slots=2, descriptor_slots=2, timeout_ms=5000, tx_warps=2, rx_warps=2,
                              output_pool_size=2)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        cases = []
        for seed in range(4):
            cpu = [make_inputs(r, world, tmax - seed * r, hidden, experts, topk, "random", seed=seed) for r in range(world)]
            dev = [tuple(t.cuda() for t in inp) for inp in cpu]
            cases.append((cpu, ([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev])))
        for epoch in range(epochs):
            cpu, args = cases[epoch % 4]
            results = group.dispatch(*args, do_expand=bool(epoch % 2))
            if epoch % 500 == 499:
                outs = group.combine([r["recv_x"] for r in results], results, weighted=False)
                torch.cuda.synchronize()
                for rank in range(world):
                    expected = reference.dispatch_reference(cpu, rank, experts, tmax, do_expand=bool(epoch % 2))
                    assert not reference.compare_dispatch(results[rank], expected, do_expand=bool(epoch % 2), do_zero_padding=False)
                del outs
            del results
        torch.cuda.synchronize()
        assert all(int(rt.sticky_error()[0]) == 0 for rt in group.runtimes)
        assert all(int(rt.epochs()[0]) == epochs for rt in group.runtimes)


def test_dispatch_and_combine_never_synchronise_the_host(ext):
    if not dist.is_initialized():
        dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="scale-store-"), 1), rank=0, world_size=1)
    torch.cuda.set_device(0)
    config = HostStagedConfig(channels=4, timeout_ms=5000)
    with HostStagedEPBuffer(None, 64, 512, 4, 16, config) as buffer:
        cpu = make_inputs(0, 1, 64, 512, 16, 4)
        x, idx, w = (t.cuda() for t in cpu)
        for _ in range(3):
            res = buffer.dispatch(x, idx, w, do_expand=True)
            out = buffer.combine(res[0], res[3])
            del res, out
        torch.cuda.synchronize()
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]) as prof:
            with torch.profiler.record_function("ep_region"):
                for _ in range(5):
                    res = buffer.dispatch(x, idx, w, do_expand=True)
                    out = buffer.combine(res[0], res[3])
                    del res, out
            torch.cuda.synchronize()
        events = prof.events()
        region = next(e for e in events if e.name == "ep_region")
        lo, hi = region.time_range.start, region.time_range.end
        inside = [e.name for e in events if e.time_range.start >= lo and e.time_range.end <= hi]
        forbidden = [n for n in inside if "Synchronize" in n or n in ("aten::item", "aten::_local_scalar_dense") or "DtoH" in n]
        assert not forbidden, forbidden
        kernels = [e.name for e in events if "dispatch_kernel" in e.name or "combine_push_kernel" in e.name]
        assert len([k for k in kernels if "dispatch_kernel" in k]) >= 5 and len([k for k in kernels if "combine_push_kernel" in k]) >= 5
        # the payload path is this library's own kernels: no NCCL kernel runs inside the region
        assert not [e.name for e in events if "nccl" in e.name.lower()]
        buffer.check_errors()
