"""The separate scatter pass (non-fused ablation) produces exactly the fused kernel's expanded layout."""

import pytest
import torch

from pcie_ep_b200.ops import reference
from pcie_ep_b200.ops.unfused_expand import scatter_expert_inputs
from tests.helpers import make_inputs


@pytest.mark.parametrize("pattern", ["random", "hotspot", "multicast", "partial", "none"])
@pytest.mark.parametrize("alignment", [1, 8])
def test_scatter_of_unique_rows_equals_the_expanded_dispatch(pattern, alignment):
    world, experts, topk, hidden, tmax = 4, 32, 4, 64, 40
    inputs = [make_inputs(r, world, [40, 17, 0, 33][r], hidden, experts, topk, pattern, seed=5) for r in range(world)]
    local = experts // world
    for rank in range(world):
        unique = reference.dispatch_reference(inputs, rank, experts, tmax, do_expand=False)
        fused = reference.dispatch_reference(inputs, rank, experts, tmax, do_expand=True, expert_alignment=alignment,
                                             do_zero_padding=True)
        capacity = fused["recv_x"].shape[0]
        out = scatter_expert_inputs(unique["recv_x"], unique["recv_topk_idx"], unique["recv_topk_weights"], unique["unique_count"],
                                    local, capacity, alignment, source_meta=unique["source_meta"])
        assert torch.equal(out["expert_counts"], fused["expert_counts"])
        assert torch.equal(out["expert_offsets"], fused["expert_offsets"])
        assert int(out["expanded_count"]) == int(fused["expanded_count"])
        assert torch.equal(out["recv_x"], fused["recv_x"])                    # padding rows are zero in both
        assert torch.equal(out["recv_topk_idx"], fused["recv_topk_idx"])
        assert torch.equal(out["recv_topk_weights"], fused["recv_topk_weights"])
        assert torch.equal(out["source_meta"], fused["source_meta"])


def test_rows_behind_the_count_and_small_results_are_handled_without_reading_back():
    x = torch.arange(12, dtype=torch.float32).reshape(6, 2)
    idx = torch.tensor([[0, 1], [1, -1], [0, -1], [1, 0], [0, 1], [0, 1]])
    out = scatter_expert_inputs(x, idx, None, torch.tensor([4]), 2, 16)      # rows 4 and 5 are beyond the count
    assert out["expert_counts"].tolist() == [3, 3] and out["expert_offsets"].tolist() == [0, 3, 6]
    assert out["recv_x"][:6, 0].tolist() == [0.0, 4.0, 6.0, 0.0, 2.0, 6.0]
    assert out["recv_topk_weights"] is None and out["recv_topk_idx"][:7].tolist() == [0, 0, 0, 1, 1, 1, -1]
    small = scatter_expert_inputs(x, idx, None, torch.tensor([4]), 2, 4)     # too small: rows are dropped, nothing is overrun
    assert small["recv_x"].shape == (4, 2) and small["recv_topk_idx"].tolist() == [0, 0, 0, 1]
    with pytest.raises(ValueError):
        scatter_expert_inputs(x, idx[:, 0], None, torch.tensor([4]), 2, 16)


def test_two_step_form_through_the_buffer_equals_its_expanded_dispatch():
    """The call sequence of benchmarks/ablation_unfused.py on the CPU transport: same handle fields, same comparison."""
    import tempfile

    import torch.distributed as dist

    from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer

    if not dist.is_initialized():
        dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(prefix="unfused-store-"), 1), rank=0, world_size=1)
    tokens, hidden, topk, experts = 16, 32, 2, 4
    g = torch.Generator().manual_seed(3)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)]).to(torch.int64)
    w = torch.rand(tokens, topk, generator=g)
    with HostStagedEPBuffer(None, tokens, hidden, topk, experts, HostStagedConfig(transport="cpu")) as buffer:
        fused = buffer.dispatch(x, idx, w, do_expand=True)
        recv_x, recv_idx, recv_w, handle, _ = buffer.dispatch(x, idx, w, do_expand=False)
        capacity = fused[0].shape[0]
        out = scatter_expert_inputs(recv_x, recv_idx, recv_w, handle.num_recv_tokens, experts, capacity)
        rows = int(out["expert_offsets"][-1])
        assert rows == tokens * topk
        assert torch.equal(fused[3].expert_counts.to(torch.int32), out["expert_counts"])
        assert torch.equal(fused[3].expert_offsets.to(torch.int32)[: experts + 1], out["expert_offsets"])
        assert torch.equal(fused[0][:rows], out["recv_x"][:rows])
        assert torch.equal(fused[2][:rows], out["recv_topk_weights"][:rows])
