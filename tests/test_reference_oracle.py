"""The vectorised oracle must agree with a token-by-token enumeration of the semantics."""

import pytest
import torch

from pcie_ep_b200.ops import reference
from tests.helpers import enumerate_reference, make_inputs


@pytest.mark.parametrize("pattern", ["random", "local", "multicast", "hotspot", "partial", "none"])
@pytest.mark.parametrize("expand,alignment", [(False, 1), (True, 1), (True, 8)])
def test_oracle_matches_enumeration(pattern, expand, alignment):
    world, experts, topk, hidden, tmax = 4, 16, 4, 16, 20
    tokens = [17, 0, 20, 5]
    inputs = [make_inputs(r, world, tokens[r], hidden, experts, topk, pattern, dtype=torch.float32) for r in range(world)]
    for rank in range(world):
        res = reference.dispatch_reference(inputs, rank, experts, tmax, do_expand=expand, expert_alignment=alignment)
        unique, expanded, counts, offsets, writes, reads, deliveries = enumerate_reference(inputs, rank, experts, alignment)
        assert int(res["unique_count"]) == len(unique)
        assert res["expert_counts"].tolist() == counts
        assert res["expert_offsets"].tolist() == offsets
        assert res["stats"][:3].tolist() == [writes, reads, deliveries]
        assert int(res["expanded_count"]) == sum(counts)
        if expand:
            for e, rows in enumerate(expanded):
                for o, (s, t, slot, w) in enumerate(rows):
                    row = offsets[e] + o
                    assert torch.equal(res["recv_x"][row], inputs[s][0][t])
                    assert int(res["recv_topk_idx"][row]) == e
                    assert float(res["recv_topk_weights"][row]) == pytest.approx(w)
                    assert res["source_meta"][row].tolist() == [s, t, slot]
                pad = slice(offsets[e] + len(rows), offsets[e + 1])
                assert not torch.count_nonzero(res["recv_x"][pad])
                assert (res["recv_topk_idx"][pad] == -1).all()
        else:
            for row, (s, t, out_idx, out_w) in enumerate(unique):
                assert torch.equal(res["recv_x"][row], inputs[s][0][t])
                assert res["recv_topk_idx"][row].tolist() == out_idx
                assert res["recv_topk_weights"][row].tolist() == pytest.approx(out_w)
                assert res["source_meta"][row].tolist() == [s, t, -1]
            offs = res["source_offsets"].tolist()
            assert offs[0] == 0 and offs[-1] == len(unique)


def test_capacities_match_reference_formula():
    assert reference.unique_capacity(8, 8192) == 65536
    assert reference.expanded_capacity(8, 8192, 8, 256) == 8 * 8192 * 8 + 32 * 255
    assert reference.expanded_capacity(8, 16, 8, 16) == 8 * 16 * 2 + 2 * 255


def test_validate_routes():
    assert reference.validate_routes(torch.tensor([[0, 1], [-1, 3]]), 4)
    assert not reference.validate_routes(torch.tensor([[0, 0]]), 4)
    assert not reference.validate_routes(torch.tensor([[0, 4]]), 4)
    assert not reference.validate_routes(torch.tensor([[-2, 1]]), 4)
    assert reference.validate_routes(torch.tensor([[-1, -1]]), 4)


def test_combine_reference_identity_expert():
    """dispatch -> identity experts -> combine gives sum_k w_k * x for every token."""
    world, experts, topk, hidden, tmax = 4, 16, 4, 32, 24
    tokens = [24, 3, 0, 11]
    inputs = [make_inputs(r, world, tokens[r], hidden, experts, topk, "random", dtype=torch.float32) for r in range(world)]
    results = [reference.dispatch_reference(inputs, r, experts, tmax, do_expand=True) for r in range(world)]
    for rank in range(world):
        out = reference.combine_reference([r["recv_x"] for r in results], results, tokens, do_expand=True, rank=rank)
        x, idx, w = inputs[rank]
        expected = x * (w * (idx >= 0)).sum(dim=1, keepdim=True)
        assert torch.allclose(out, expected, rtol=1e-5, atol=1e-5)
