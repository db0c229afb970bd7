"""Fused down-projection + combine: the tcgen05 GEMM's epilogue writes weighted rows straight into the token
owners' landing slots (peer pointers in the same kernel as the tensor-core tiles), the owners add their K slots.
Checked against the two-step path (grouped GEMM, then the combine kernel) and against a dense FP32 evaluation,
over several epochs with changing routes; the bounded wait is exercised with a rank whose GEMM never runs."""

import pytest
import torch

from pcie_ep_b200 import HostStagedConfig
from pcie_ep_b200.ops.grouped_ffn import grouped_gemm
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


def _weights(world, local, hidden, inter, seed=0):
    gen = torch.Generator().manual_seed(seed)
    w13 = [(torch.randn(local, 2 * inter, hidden, generator=gen) * 0.05).to(torch.bfloat16).cuda() for _ in range(world)]
    w2 = [(torch.randn(local, hidden, inter, generator=gen) * 0.05).to(torch.bfloat16).cuda() for _ in range(world)]
    return w13, w2


def _dense(x, idx, w, w13, w2, local, inter):
    out = torch.zeros(x.shape[0], x.shape[1])
    xf = x.float()
    for e in torch.unique(idx[idx >= 0]).tolist():
        a, b = w13[e // local][e % local].float().cpu(), w2[e // local][e % local].float().cpu()
        tokens, slots = torch.nonzero(idx == e, as_tuple=True)
        full = xf[tokens] @ a.t()
        h = (torch.nn.functional.silu(full[:, :inter]) * full[:, inter:]).to(torch.bfloat16).float()
        out.index_add_(0, tokens, (h @ b.t()) * w[tokens, slots].unsqueeze(1))
    return out


@pytest.mark.parametrize("alignment", [1, 16])
def test_fused_expert_combine_matches_two_step_path_and_dense_reference(ext, alignment):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, inter, tmax = 4, 16, 4, 512, 256, 96
    local = experts // world
    config = HostStagedConfig(channels=4, timeout_ms=5000, fused_expert_combine=True)
    w13, w2 = _weights(world, local, hidden, inter)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for epoch in range(3):
            cpu = [make_inputs(r, world, tmax - 7 * r - epoch, hidden, experts, topk, "random", seed=epoch) for r in range(world)]
            for inp in cpu:
                inp[0][:, :2] *= 0.01  # the helper's token-identity columns are large: keep the activations O(1)
            if epoch == 1:  # unused slots must be skipped by the owner
                for inp in cpu:
                    inp[1][::3, 1] = -1
            dev = [tuple(t.cuda() for t in inp) for inp in cpu]
            results = group.dispatch([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], do_expand=True,
                                     expert_alignment=alignment)
            hid, status = [], torch.zeros(4, dtype=torch.int32, device="cuda")
            for r in range(world):
                rows = results[r]["recv_x"]
                h = torch.zeros(rows.shape[0], inter, dtype=torch.bfloat16, device="cuda")
                grouped_gemm(rows, w13[r], results[r]["expert_offsets"], results[r]["expert_counts"], swiglu=True, out=h, status=status)
                hid.append(h)
            fused = [t.clone() for t in group.fused_expert_combine(hid, w2, results)]
            ys = []
            for r in range(world):
                y = torch.zeros(hid[r].shape[0], hidden, dtype=torch.bfloat16, device="cuda")
                grouped_gemm(hid[r], w2[r], results[r]["expert_offsets"], results[r]["expert_counts"], swiglu=False, out=y, status=status)
                ys.append(y)
            two_step = group.combine(ys, results, weighted=True)
            torch.cuda.synchronize()
            assert status.tolist()[0] == 0
            for r in range(world):
                assert int(group.runtimes[r].fused_status()[0]) == 0
                assert results[r]["combine_error"].tolist()[0] == 0
                want = _dense(cpu[r][0], cpu[r][1], cpu[r][2], w13, w2, local, inter)
                got = fused[r].float().cpu()
                assert got.shape == want.shape
                assert torch.allclose(got, want, rtol=3e-2, atol=3e-2), (epoch, r, (got - want).abs().max())
                assert torch.allclose(got, two_step[r].float().cpu(), rtol=2e-2, atol=2e-2)
            del results, two_step


def test_fused_reduce_gives_up_when_a_rank_never_signals(ext):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, inter, tmax = 2, 4, 2, 256, 128, 16
    config = HostStagedConfig(channels=2, timeout_ms=300, fused_expert_combine=True)
    w13, w2 = _weights(world, experts // world, hidden, inter)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        cpu = [make_inputs(r, world, tmax, hidden, experts, topk, "random", seed=5) for r in range(world)]
        dev = [tuple(t.cuda() for t in inp) for inp in cpu]
        results = group.dispatch([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], do_expand=True)
        hid = [torch.zeros(results[r]["recv_x"].shape[0], inter, dtype=torch.bfloat16, device="cuda") for r in range(world)]
        group.fused_expert_combine(hid, w2, results, ranks=[0])  # rank 1's GEMM never runs: nothing sets its flag
        torch.cuda.synchronize()
        error = results[0]["combine_error"].tolist()
        assert error[0] == 25 and error[1] == 1, error
        assert int(group.runtimes[0].sticky_error()[0]) == 25
        # the context survives: a plain kernel still runs
        assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def test_fused_expert_combine_needs_the_option(ext):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    with VirtualEPGroup(2, 16, 256, 2, 4, HostStagedConfig(channels=2, timeout_ms=2000)) as group:
        cpu = [make_inputs(r, 2, 16, 256, 4, 2, "random", seed=1) for r in range(2)]
        dev = [tuple(t.cuda() for t in inp) for inp in cpu]
        results = group.dispatch([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], do_expand=True)
        hid = [torch.zeros(results[r]["recv_x"].shape[0], 128, dtype=torch.bfloat16, device="cuda") for r in range(2)]
        w2 = [torch.zeros(2, 256, 128, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        with pytest.raises(RuntimeError, match="fused_expert_combine=False"):
            group.fused_expert_combine(hid, w2, results)
