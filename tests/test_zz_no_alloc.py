"""The allocation-free routing-layout entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory where they need a routing plan: a server
that carved up all of its memory at start-up, a plugin living inside another framework's allocator,
or a section where cudaMalloc's device-wide synchronisation is unacceptable.  For them
``bep_route_layout_static`` keeps its cross-CTA scratch in an array inside the loaded library.  This
test calls it twice in a row (different routes, different token counts, so anything left in the
shared scratch by the first call would show) and requires, both times, exactly the plan that a
regular dispatch computes for the same routes.  The plan is integer data, so the comparison is exact.
"""

import ctypes

import pytest
import torch

from pcie_ep_b200 import HostStagedConfig
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


def _entry(ext):
    lib = ctypes.CDLL(str(ext._library_path()))
    fn = lib.bep_route_layout_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.bep_route_layout_static_scratch_bytes.restype = ctypes.c_ulonglong
    return lib, fn


def test_static_layout_matches_dispatch_plan_twice(ext):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    lib, fn = _entry(ext)
    assert lib.bep_route_layout_static_scratch_bytes() == 266496
    world, experts, topk, hidden, tmax, channels = 4, 64, 4, 128, 96, 8
    config = HostStagedConfig(channels=channels, timeout_ms=2000, tx_warps=2, rx_warps=2)
    stream = torch.cuda.current_stream()
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for call, (tokens, pattern, seed) in enumerate([(96, "random", 3), (41, "partial", 11)]):
            inputs = [tuple(None if t is None else t.cuda() for t in
                            make_inputs(r, world, tokens, hidden, experts, topk, pattern, seed=seed))
                      for r in range(world)]
            results = group.dispatch([i[0] for i in inputs], [i[1] for i in inputs], [i[2] for i in inputs],
                                     do_expand=True)
            torch.cuda.synchronize()
            for rank in (0, world - 1):
                plan = results[rank]["_layout"]
                idx = inputs[rank][1]
                # outputs are the caller's; poison them so untouched words would show
                mask = torch.full((tmax,), -7, dtype=torch.int32, device="cuda")
                slot = torch.full((tmax, world), -7, dtype=torch.int32, device="cuda")
                order = torch.full((tmax, topk), -7, dtype=torch.int32, device="cuda")
                counts = torch.full((world + experts + channels * world,), -7, dtype=torch.int32, device="cuda")
                status = torch.full((4,), -7, dtype=torch.int32, device="cuda")
                rc = fn(idx.data_ptr(), tokens, topk, experts, world, channels, mask.data_ptr(), slot.data_ptr(),
                        order.data_ptr(), counts.data_ptr(), status.data_ptr(), stream.cuda_stream)
                assert rc == 0, f"call {call}: entry point returned {rc}"
                torch.cuda.synchronize()
                assert status.tolist() == [0, 0, 0, 0]
                assert torch.equal(mask[:tokens], plan.mask[:tokens]), f"call {call} rank {rank}: mask"
                assert torch.equal(slot[:tokens], plan.slot[:tokens]), f"call {call} rank {rank}: slot"
                assert torch.equal(order[:tokens], plan.expert_ord[:tokens]), f"call {call} rank {rank}: ordinals"
                assert torch.equal(counts, plan.counts), f"call {call} rank {rank}: counts"
            del results, plan


def test_static_layout_rejects_oversize_and_bad_arguments(ext):
    _, fn = _entry(ext)
    dummy = torch.zeros(64, dtype=torch.int64, device="cuda")
    out = torch.zeros(4096, dtype=torch.int32, device="cuda")
    args = (dummy.data_ptr(), 4, 2, 8, 2, 2, out.data_ptr(), out.data_ptr(), out.data_ptr(), out.data_ptr(),
            out.data_ptr(), 0)
    too_many_channels = list(args)
    too_many_channels[5] = 65
    assert fn(*too_many_channels) == -1
    too_many_experts = list(args)
    too_many_experts[3] = 2048
    assert fn(*too_many_experts) == -1
    uneven = list(args)
    uneven[3] = 9
    assert fn(*uneven) == -2
    null_status = list(args)
    null_status[10] = None
    assert fn(*null_status) == -2
    torch.cuda.synchronize()


def test_static_layout_reports_invalid_routes_and_handles_edge_sizes(ext):
    """A repeated or out-of-range expert id is reported through `status` ([2, token, slot, 0]); zero tokens and more
    channels than tokens are ordinary requests."""
    _, fn = _entry(ext)
    experts, ranks, topk, channels, tokens = 16, 2, 4, 4, 9
    stream = torch.cuda.current_stream().cuda_stream

    def run(idx, tokens, channels):
        mask = torch.full((max(tokens, 1),), -7, dtype=torch.int32, device="cuda")
        slot = torch.full((max(tokens, 1), ranks), -7, dtype=torch.int32, device="cuda")
        order = torch.full((max(tokens, 1), topk), -7, dtype=torch.int32, device="cuda")
        counts = torch.full((ranks + experts + channels * ranks,), -7, dtype=torch.int32, device="cuda")
        status = torch.full((4,), -7, dtype=torch.int32, device="cuda")
        rc = fn(idx.data_ptr() if tokens else None, tokens, topk, experts, ranks, channels,
                mask.data_ptr() if tokens else None, slot.data_ptr() if tokens else None,
                order.data_ptr() if tokens else None, counts.data_ptr(), status.data_ptr(), stream)
        torch.cuda.synchronize()
        return rc, status.tolist(), counts, mask

    base = torch.stack([torch.randperm(experts)[:topk] for _ in range(tokens)]).to(torch.int64)
    duplicate = base.clone()
    duplicate[5, 2] = duplicate[5, 0]
    rc, status, _, _ = run(duplicate.cuda(), tokens, channels)
    assert rc == 0 and status == [2, 5, 2, 0]
    out_of_range = base.clone()
    out_of_range[7, 1] = experts
    rc, status, _, _ = run(out_of_range.cuda(), tokens, channels)
    assert rc == 0 and status == [2, 7, 1, 0]
    # no tokens at all: per-token arrays may be null, every count is zero
    rc, status, counts, _ = run(base.cuda(), 0, channels)
    assert rc == 0 and status == [0, 0, 0, 0] and int(counts.abs().sum()) == 0
    # more channels than tokens: same totals as with one channel
    rc_many, status_many, counts_many, mask_many = run(base.cuda(), tokens, 16)
    rc_one, status_one, counts_one, mask_one = run(base.cuda(), tokens, 1)
    assert rc_many == 0 and rc_one == 0 and status_many == [0, 0, 0, 0] and status_one == [0, 0, 0, 0]
    assert torch.equal(counts_many[:ranks + experts], counts_one[:ranks + experts]) and torch.equal(mask_many, mask_one)
