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
