"""The two-step form of an expanded dispatch on the GPU: a unique dispatch of the fused kernel followed by the separate
scatter pass (device-side tensor operations) gives, row for row, what the fused receive + expand produces."""

import pytest
import torch

from pcie_ep_b200 import HostStagedConfig
from pcie_ep_b200.ops.unfused_expand import scatter_expert_inputs
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("alignment", [1, 16])
def test_unique_dispatch_plus_scatter_pass_equals_the_fused_expansion(ext, alignment):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 32, 4, 256, 40
    local = experts // world
    config = HostStagedConfig(channels=4, timeout_ms=2000, tx_warps=2, rx_warps=3, output_pool_size=3)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        cpu = [make_inputs(r, world, [40, 17, 0, 33][r], hidden, experts, topk, "random", seed=21) for r in range(world)]
        dev = [tuple(t.cuda() for t in inp) for inp in cpu]
        args = ([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev])
        fused = group.dispatch(*args, do_expand=True, expert_alignment=alignment, do_zero_padding=True)
        unique = group.dispatch(*args, do_expand=False)
        torch.cuda.synchronize()
        for rank in range(world):
            f, u = fused[rank], unique[rank]
            out = scatter_expert_inputs(u["recv_x"], u["recv_topk_idx"], u["recv_topk_weights"], u["unique_count"], local,
                                        f["recv_x"].shape[0], alignment, source_meta=u["source_meta"])
            assert out["recv_x"].is_cuda
            rows = int(f["expert_offsets"].reshape(-1)[local])
            assert torch.equal(out["expert_counts"], f["expert_counts"].reshape(-1).to(torch.int32))
            assert torch.equal(out["expert_offsets"], f["expert_offsets"].reshape(-1)[: local + 1].to(torch.int32))
            assert torch.equal(out["recv_x"][:rows], f["recv_x"][:rows])                      # padding rows: zero in both
            assert torch.equal(out["recv_topk_idx"][:rows], f["recv_topk_idx"].reshape(-1)[:rows].to(out["recv_topk_idx"].dtype))
            assert torch.equal(out["recv_topk_weights"][:rows], f["recv_topk_weights"].reshape(-1)[:rows])
            assert torch.equal(out["source_meta"][:rows], f["source_meta"][:rows])
