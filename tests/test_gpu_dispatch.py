"""Fused dispatch kernel against the PyTorch oracle, several ranks emulated on one GPU in one
cooperative launch.  Coverage follows the reference's correctness matrix
(tests/test_correctness.py:228-262): patterns random/local/multicast/hotspot/partial/none, unique and
expanded layouts, zero and unequal token counts, alignment with zero padding, no weights, tiny rings."""

import pytest
import torch

from pcie_ep_b200 import HostStagedConfig
from pcie_ep_b200.ops import reference
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


def _run_case(group, world, experts, topk, hidden, tmax, tokens, pattern, expand, alignment, weights=True, seed=7,
              wire="bf16", zero_padding=None, recv="bf16"):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup  # noqa: F401

    cpu_inputs = [make_inputs(r, world, tokens[r], hidden, experts, topk, pattern, seed=seed, weights=weights)
                  for r in range(world)]
    dev = [tuple(None if t is None else t.cuda() for t in inp) for inp in cpu_inputs]
    zero_padding = expand if zero_padding is None else zero_padding
    results = group.dispatch([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], do_expand=expand,
                             expert_alignment=alignment, do_zero_padding=zero_padding)
    torch.cuda.synchronize()
    for rank in range(world):
        expected = reference.dispatch_reference(cpu_inputs, rank, experts, tmax, do_expand=expand,
                                                expert_alignment=alignment, do_zero_padding=zero_padding,
                                                wire_dtype=wire, recv_dtype=recv)
        problems = reference.compare_dispatch(results[rank], expected, do_expand=expand,
                                              do_zero_padding=zero_padding, have_weights=weights)
        assert not problems, f"rank {rank} pattern={pattern} expand={expand}: {problems}"
    return results, cpu_inputs


@pytest.mark.parametrize("engine", ["vector", "tma"])
def test_dispatch_patterns(ext, engine):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 32, 4, 256, 40
    config = HostStagedConfig(channels=4, copy_engine=engine, timeout_ms=2000, tx_warps=2, rx_warps=3)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        assert group.runtimes[0].uses_tma() == (engine == "tma")
        for pattern in ["random", "local", "multicast", "hotspot", "partial", "none"]:
            for expand in (False, True):
                _run_case(group, world, experts, topk, hidden, tmax, [17] * world, pattern, expand, 1)
        _run_case(group, world, experts, topk, hidden, tmax, [0] * world, "random", True, 1)
        _run_case(group, world, experts, topk, hidden, tmax, [0, 40, 37, 1], "random", True, 1)
        _run_case(group, world, experts, topk, hidden, tmax, [33] * world, "random", True, 16)
        _run_case(group, world, experts, topk, hidden, tmax, [5] * world, "multicast", True, 1, weights=False)
        for i in range(6):
            _run_case(group, world, experts, topk, hidden, tmax, [3 + i % 5] * world, "random", bool(i % 2), 8,
                      seed=100 + i)


def test_dispatch_odd_hidden_scalar_path(ext):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 2, 8, 2, 129, 20
    config = HostStagedConfig(channels=2, timeout_ms=2000, tx_warps=2, rx_warps=2)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        assert not group.runtimes[0].uses_tma()
        for expand in (False, True):
            _run_case(group, world, experts, topk, hidden, tmax, [19, 20], "random", expand, 1)


@pytest.mark.parametrize("engine", ["vector", "tma"])
@pytest.mark.parametrize("slots", [1, 2, 3])
def test_dispatch_tiny_rings(ext, engine, slots):
    """Bounded rings: rows wait for ACK credit (reference windows (1,1),(2,3),(3,2))."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 32, 4, 128, 48
    config = HostStagedConfig(channels=2, payload_slots=slots, descriptor_slots=slots, copy_engine=engine,
                              timeout_ms=2000, tx_warps=2, rx_warps=2)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for epoch in range(3):
            res, _ = _run_case(group, world, experts, topk, hidden, tmax, [48, 31, 0, 48], "random", True, 1,
                               seed=20 + epoch)
            del res


@pytest.mark.parametrize("engine", ["vector", "tma"])
def test_dispatch_fp8_wire(ext, engine):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 32, 4, 512, 32
    config = HostStagedConfig(channels=4, stage=7, wire_dtype="fp8_e4m3", copy_engine=engine, timeout_ms=2000,
                              tx_warps=2, rx_warps=3)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for expand in (False, True):
            _run_case(group, world, experts, topk, hidden, tmax, [32, 7, 19, 32], "random", expand, 1, wire="fp8_e4m3")


@pytest.mark.parametrize("engine", ["vector", "tma"])
def test_dispatch_fp8_rows_stay_fp8_at_the_receiver(ext, engine):
    """recv_dtype=fp8_e4m3: every row (local too) arrives as E4M3 codes plus one scale per row."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 32, 4, 512, 32
    config = HostStagedConfig(channels=4, stage=7, wire_dtype="fp8_e4m3", recv_dtype="fp8_e4m3", copy_engine=engine,
                              timeout_ms=2000, tx_warps=2, rx_warps=3)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for expand, alignment in ((False, 1), (True, 1), (True, 8)):
            results, _ = _run_case(group, world, experts, topk, hidden, tmax, [32, 7, 19, 32], "random", expand, alignment,
                                   wire="fp8_e4m3", recv="fp8_e4m3")
            assert results[0]["recv_x"].dtype == torch.float8_e4m3fn
            del results


@pytest.mark.parametrize("engine", ["vector", "tma"])
@pytest.mark.parametrize("recv", ["bf16", "fp8_e4m3"])
def test_dispatch_fp8_corner_rows(ext, engine, recv):
    """Rows that sit on the edges of the E4M3 wire format go through the kernel's own quantisation (send warps and
    the local path) and come out exactly as the PyTorch reference of the format says: an all-zero row (scale 1), a
    row whose largest magnitude is exactly 448 (scale 1), a negative extreme, a row with one element 50 times the
    rest, a row of tiny values whose scaled codes are subnormal, and a row that mixes all of these."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 16, 4, 512, 32
    tokens = [32, 9, 20, 32]
    config = HostStagedConfig(channels=4, stage=7, wire_dtype="fp8_e4m3", recv_dtype=recv, copy_engine=engine, timeout_ms=2000,
                              tx_warps=2, rx_warps=3)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for expand in (True, False):
            cpu_inputs = [list(make_inputs(r, world, tokens[r], hidden, experts, topk, "random", seed=11)) for r in range(world)]
            for r, inp in enumerate(cpu_inputs):
                x = inp[0].float()
                x[0] = 0.0
                x[1] = torch.linspace(-1.0, 1.0, hidden) * 448.0
                x[2] = -x[2].abs() - 1.0
                x[2, 7] = -30000.0
                x[3, r] = x[3].abs().max() * 50.0
                x[4] = torch.randn(hidden) * 1e-30
                x[5, ::2] = 0.0
                x[5, 1] = 448.0
                x[5, 3] = -1e-3
                inp[0] = x.to(torch.bfloat16)
            cpu_inputs = [tuple(inp) for inp in cpu_inputs]
            dev = [tuple(None if t is None else t.cuda() for t in inp) for inp in cpu_inputs]
            results = group.dispatch([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], do_expand=expand,
                                     expert_alignment=1, do_zero_padding=expand)
            torch.cuda.synchronize()
            for rank in range(world):
                expected = reference.dispatch_reference(cpu_inputs, rank, experts, tmax, do_expand=expand, expert_alignment=1,
                                                        do_zero_padding=expand, wire_dtype="fp8_e4m3", recv_dtype=recv)
                problems = reference.compare_dispatch(results[rank], expected, do_expand=expand, do_zero_padding=expand,
                                                      have_weights=True)
                assert not problems, f"rank {rank} expand={expand}: {problems}"


def test_dispatch_headline_shape_small_t(ext):
    """DeepSeek-V3 shape (hidden 7168, 256 experts, top-8) at small T on 8 emulated ranks."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 8, 256, 8, 7168, 64
    config = HostStagedConfig(channels=8, timeout_ms=5000, tx_warps=4, rx_warps=8)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        assert group.runtimes[0].uses_tma()
        results, inputs = _run_case(group, world, experts, topk, hidden, tmax, [64] * world, "random", True, 1)
        # dedup counters equal the route volume
        for rank in range(world):
            volume = reference.route_volume(inputs[rank][1], rank, world, experts)
            stats = results[rank]["stats"].cpu().tolist()
            assert stats[0] == volume["remote_source_tokens"]
            assert stats[2] == volume["remote_deliveries"]


@pytest.mark.parametrize("send_ctas", [0, 4])
def test_dispatch_headline_shape_four_ranks_many_channels(ext, send_ctas):
    """Four emulated ranks with 32 channels each (two groups of the layout's two-level prefix, several sources per
    receive warp, rows with up to three remote destinations), with the send warps inside the channel CTAs and with
    dedicated sender CTAs; repeated, so that the layout's alternating scratch is used on both sides."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 256, 8, 7168, 128
    config = HostStagedConfig(channels=32, timeout_ms=5000, tx_warps=2 if send_ctas == 0 else 4, rx_warps=8, send_ctas=send_ctas,
                              output_pool_size=2)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for repeat in range(4):
            results, inputs = _run_case(group, world, experts, topk, hidden, tmax, [128, 128, 97, 128], "random", True, 1,
                                        seed=7 + repeat)
            for rank in range(world):
                volume = reference.route_volume(inputs[rank][1], rank, world, experts)
                stats = results[rank]["stats"].cpu().tolist()
                assert stats[0] == volume["remote_source_tokens"]
                assert stats[2] == volume["remote_deliveries"]
            del results


def test_pool_exhaustion_and_release(ext):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 2, 8, 2, 64, 8
    config = HostStagedConfig(channels=1, output_pool_size=2, timeout_ms=2000, tx_warps=1, rx_warps=1)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        inputs = [tuple(t.cuda() for t in make_inputs(r, world, 8, hidden, experts, topk)) for r in range(world)]
        args = ([i[0] for i in inputs], [i[1] for i in inputs], [i[2] for i in inputs])
        first = group.dispatch(*args, do_expand=True)
        second = group.dispatch(*args, do_expand=True)
        with pytest.raises(RuntimeError, match="pool exhausted"):
            group.dispatch(*args, do_expand=True)
        keep = first[0]["expert_counts"]  # a single small tensor keeps its whole set busy
        del first
        with pytest.raises(RuntimeError, match="pool exhausted"):
            group.dispatch(*args, do_expand=True)
        del keep
        third = group.dispatch(*args, do_expand=True)
        torch.cuda.synchronize()
        assert all(int(r["error"][0]) == 0 for r in third)
        del second, third


@pytest.mark.parametrize("mode", ["separate", "inline"])
def test_combine_modes_on_emulated_ranks(ext, mode):
    """Owner-side sum as a second launch ("separate") or inside the cooperative kernel ("inline"): both return
    x * (sum of the token's weights) for identity experts, over epochs with changing routes, unequal token
    counts, unused slots and the unique layout."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    world, experts, topk, hidden, tmax = 4, 16, 4, 512, 48
    config = HostStagedConfig(channels=4, timeout_ms=3000, tx_warps=2, rx_warps=3, combine_reduce=mode)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for epoch in range(5):
            tokens = [tmax - 5 * r - epoch for r in range(world)]
            if epoch == 3:
                tokens[1] = 0
            expand = epoch != 2
            pattern = "partial" if epoch == 1 else "random"
            cpu = [make_inputs(r, world, tokens[r], hidden, experts, topk, pattern, seed=10 + epoch) for r in range(world)]
            dev = [tuple(t.cuda() for t in inp) for inp in cpu]
            results = group.dispatch([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev], do_expand=expand)
            outs = group.combine([r["recv_x"] for r in results], results, weighted=expand)
            torch.cuda.synchronize()
            local = experts // world
            for r in range(world):
                assert results[r]["combine_error"].tolist()[0] == 0, results[r]["combine_error"].tolist()
                x, idx, w = cpu[r]
                if expand:
                    scale = (w * (idx >= 0)).sum(dim=1, keepdim=True)
                else:  # unique layout, unweighted: one copy per destination rank
                    ranks = torch.where(idx >= 0, idx // local, torch.full_like(idx, -1))
                    scale = torch.stack([(ranks == d).any(dim=1) for d in range(world)], dim=1).sum(dim=1, keepdim=True).float()
                want = x.float() * scale
                got = outs[r].cpu().float()
                assert got.shape == want.shape
                assert torch.allclose(got, want, rtol=2e-2, atol=2e-2), (mode, epoch, r, (got - want).abs().max())
            del results, outs
        assert all(int(rt.sticky_error()[0]) == 0 for rt in group.runtimes)
