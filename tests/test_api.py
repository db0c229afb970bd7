"""API contracts that need no GPU (reference: tests/test_api.py): export identity, EventOverlap semantics,
handle aliases and route guards, argument rejections, cached-layout validation, collective error
agreement, NCCL borrow without an NCCL group -- exercised on the CPU transport in-process (world size 1)."""

import tempfile

import pytest
import torch
import torch.distributed as dist

import pcie_ep_b200
from pcie_ep_b200 import (CachedLayout, EPBuffer, EPHandle, EventOverlap, HostStagedConfig, HostStagedEPBuffer,
                          HostStagedEPHandle, topk_idx_t)
from pcie_ep_b200.parallel import control


@pytest.fixture(scope="module")
def world1():
    if not dist.is_initialized():
        store = dist.FileStore(tempfile.mktemp(prefix="api-store-"), 1)
        dist.init_process_group("gloo", store=store, rank=0, world_size=1)
    yield
    # left initialised for other in-process tests of this module


@pytest.fixture()
def buffer(world1):
    buf = HostStagedEPBuffer(None, 16, 32, 2, 4, HostStagedConfig(transport="cpu", enable_graph=True))
    yield buf
    buf.close()


def _inputs(tokens=5, hidden=32, topk=2, experts=4):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(tokens, hidden, generator=g)
    idx = torch.rand(tokens, experts, generator=g).topk(topk, dim=1).indices.to(torch.int64)
    w = torch.rand(tokens, topk, generator=g)
    return x, idx, w


def test_export_identity():
    import pcie_ep_b200.buffer as legacy

    assert EPBuffer is HostStagedEPBuffer and EPHandle is HostStagedEPHandle
    assert legacy.HostStagedEPBuffer is HostStagedEPBuffer and legacy.EventOverlap is EventOverlap
    assert topk_idx_t is torch.int64
    assert set(pcie_ep_b200.__all__) >= {"HostStagedConfig", "HostStagedEPBuffer", "HostStagedEPHandle",
                                         "CachedLayout", "GraphDispatch", "EventOverlap", "topk_idx_t"}


def test_constructor_requires_initialised_distributed(monkeypatch):
    monkeypatch.setattr(dist, "is_initialized", lambda: False)
    with pytest.raises(RuntimeError, match="Initialize torch.distributed"):
        HostStagedEPBuffer(None, 4, 8, 2, 4)


def test_constructor_argument_checks(world1):
    with pytest.raises(ValueError, match="not both"):
        HostStagedEPBuffer(None, 4, 8, 2, 4, HostStagedConfig(transport="cpu"), host_staged_config=HostStagedConfig())
    with pytest.raises(ValueError, match="positive integer"):
        HostStagedEPBuffer(None, 0, 8, 2, 4, HostStagedConfig(transport="cpu"))
    with pytest.raises(ValueError, match="transport"):
        HostStagedEPBuffer(None, 4, 8, 2, 4, transport="smoke-signals")
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="requires NVIDIA CUDA"):
            HostStagedEPBuffer(None, 4, 8, 2, 4, transport="peer")


def test_dispatch_returns_five_items_and_handle_aliases(buffer):
    x, idx, w = _inputs()
    recv_x, recv_idx, recv_w, handle, event = buffer.dispatch(x, idx, w, do_expand=True)
    assert isinstance(handle, HostStagedEPHandle) and isinstance(event, EventOverlap)
    assert recv_x.shape[1] == 32 and recv_idx.ndim == 1 and recv_w.ndim == 1
    assert handle.num_recv_tokens is handle.unique_count
    assert handle.num_expanded_tokens is handle.expanded_count
    assert handle.num_unaligned_recv_tokens_per_expert is handle.expert_counts
    assert handle.recv_src_metadata is handle.source_meta
    assert torch.equal(handle.psum_num_recv_tokens_per_scaleup_rank, handle.source_offsets[1:])
    assert torch.equal(handle.psum_num_recv_tokens_per_expert, handle.expert_offsets[:-1] + handle.expert_counts)
    assert handle.num_recv_tokens_per_expert_list is None and handle.num_sms == 0
    assert int(handle.unique_count) == 5 and int(handle.expanded_count) == 10
    handle.check_errors()
    # without weights the third item is None
    assert buffer.dispatch(x, idx, do_expand=False)[2] is None


@pytest.mark.parametrize("overrides,error", [
    (dict(do_cpu_sync=True), NotImplementedError),
    (dict(do_handle_copy=True), NotImplementedError),
    (dict(num_qps=1), NotImplementedError),
    (dict(num_sms=4), NotImplementedError),
    (dict(use_tma_aligned_col_major_sf=True), NotImplementedError),
    (dict(previous_event=object()), ValueError),
    (dict(defer_epilogue=True), ValueError),
    (dict(do_zero_padding=True, do_expand=False), ValueError),
    (dict(expert_alignment=0), ValueError),
    (dict(expert_alignment=1.5), ValueError),
    (dict(num_experts=5), ValueError),
    (dict(num_max_tokens_per_rank=17), ValueError),
])
def test_dispatch_rejections(buffer, overrides, error):
    x, idx, w = _inputs()
    kwargs = dict(x=x, topk_idx=idx, topk_weights=w)
    kwargs.update(overrides)
    with pytest.raises(error):
        buffer.dispatch(**kwargs)


def test_dispatch_input_validation(buffer):
    x, idx, w = _inputs()
    with pytest.raises(TypeError):
        buffer.dispatch([1, 2], idx)
    with pytest.raises(ValueError):
        buffer.dispatch(x[:, :-1], idx)                       # wrong hidden
    with pytest.raises(ValueError):
        buffer.dispatch(x, idx[:, :-1].contiguous())          # wrong top-k
    with pytest.raises(ValueError):
        buffer.dispatch(x, idx.to(torch.int32))               # wrong dtype
    with pytest.raises(ValueError):
        buffer.dispatch(x, idx, w[:, :-1].contiguous())
    with pytest.raises(ValueError):
        buffer.dispatch(x.t().contiguous().t(), idx)          # non-contiguous
    with pytest.raises(ValueError):
        buffer.dispatch(torch.randn(17, 32), torch.zeros(17, 2, dtype=torch.int64))  # over capacity
    with pytest.raises(ValueError):
        buffer.dispatch(x, idx, handle=object())              # handle and topk_idx together


def test_defer_epilogue_returns_outputs_once(buffer):
    x, idx, w = _inputs()
    overlap = buffer.dispatch(x, idx, w, async_with_compute_stream=True, defer_epilogue=True)
    assert isinstance(overlap, EventOverlap)
    first = overlap.wait()
    assert isinstance(first, tuple) and len(first) == 4 and isinstance(first[3], HostStagedEPHandle)
    assert overlap.wait() is None


def test_event_overlap_semantics():
    calls = []
    overlap = EventOverlap(None, ("refs",), on_wait=lambda stream: calls.append(stream))
    overlap.register_hook_after_wait(lambda: "payload")
    with pytest.raises(RuntimeError):
        overlap.register_hook_after_wait(lambda: "again")
    assert overlap.current_stream_wait() == "payload"
    assert overlap.wait() is None
    with overlap(release_handle=True):
        pass
    with pytest.raises(RuntimeError, match="released"):
        overlap.wait()
    with overlap:  # released events exit quietly
        pass


def test_route_guard_and_cached_layout(buffer):
    x, idx, w = _inputs()
    _, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=True, expert_alignment=4)
    cache = buffer.cache_layout(handle)
    assert isinstance(cache, CachedLayout) and not hasattr(cache, "_result")
    again = buffer.dispatch(x * 2, topk_weights=w, handle=cache, do_expand=True)
    assert again[3].expert_alignment == 4
    with pytest.raises(ValueError, match="alignment or expansion"):
        buffer.dispatch(x, handle=cache, do_expand=False)
    with pytest.raises(ValueError):  # the token count no longer matches the cached routes
        buffer.dispatch(x[:3].contiguous(), handle=cache, do_expand=True)
    idx.add_(0)  # bumps the version counter
    with pytest.raises(RuntimeError, match="topk_idx changed"):
        buffer.dispatch(x, handle=cache, do_expand=True)
    with pytest.raises(RuntimeError, match="topk_idx changed"):
        handle.topk_idx


def test_cached_layout_needs_version_counter(buffer):
    x, idx, w = _inputs()
    with torch.inference_mode():
        frozen = idx.clone()
    handle = buffer.dispatch(x, frozen, w)[3]
    with pytest.raises(ValueError, match="version counter"):
        buffer.cache_layout(handle)


def test_handles_are_tied_to_their_buffer(world1):
    a = HostStagedEPBuffer(None, 16, 32, 2, 4, HostStagedConfig(transport="cpu"))
    b = HostStagedEPBuffer(None, 16, 32, 2, 4, HostStagedConfig(transport="cpu"))
    x, idx, w = _inputs()
    handle = a.dispatch(x, idx, w)[3]
    with pytest.raises(ValueError):
        b.check_errors(handle)
    with pytest.raises(ValueError):
        b.cache_layout(handle)
    with pytest.raises(ValueError):
        b.combine(x, handle)
    a.close()
    b.close()
    with pytest.raises(RuntimeError, match="closed"):
        a.dispatch(x, idx, w)
    a.close()  # idempotent


def test_invalid_routes_fail_the_buffer(world1):
    buf = HostStagedEPBuffer(None, 16, 32, 2, 4, HostStagedConfig(transport="cpu"))
    x, idx, w = _inputs()
    bad = idx.clone()
    bad[0, 1] = bad[0, 0]
    buf.dispatch(x, bad, w)
    with pytest.raises(RuntimeError, match="GPU error"):
        buf.check_errors()
    with pytest.raises(RuntimeError, match="failed"):
        buf.dispatch(x, idx, w)
    buf.close()


def test_combine_round_trip_and_rejections(buffer):
    x, idx, w = _inputs()
    recv_x, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=True)
    combined, _, event = buffer.combine(recv_x, handle)
    event.wait()
    assert torch.allclose(combined, x * w.sum(dim=1, keepdim=True), rtol=1e-5, atol=1e-5)
    with pytest.raises(TypeError):
        buffer.combine(recv_x, object())
    with pytest.raises(NotImplementedError):
        buffer.combine(recv_x, handle, topk_weights=w)
    with pytest.raises(ValueError):
        buffer.combine(recv_x, handle, previous_event=object())


def test_capture_dispatch_needs_a_gpu_transport(buffer):
    x, idx, w = _inputs()
    with pytest.raises(NotImplementedError):
        buffer.capture_dispatch(x, idx, w)


def test_nccl_borrow_without_nccl_group(world1):
    borrowed = control.borrow_nccl_comm(dist.group.WORLD, "cpu")
    assert borrowed.nccl_comm is None and not borrowed.reused and borrowed.status == "not_an_nccl_group"
    with pytest.raises(RuntimeError):
        control.borrow_nccl_comm(dist.group.WORLD, "cpu", require_reuse=True)


def test_control_group_rules_and_agreement(world1):
    group, owned = control.get_control_group(dist.group.WORLD, (0,))
    assert group is dist.group.WORLD and not owned
    with pytest.raises(ValueError):
        control.get_control_group(dist.group.WORLD, (0, 1), control_group=dist.group.WORLD)
    control.agree(None, dist.group.WORLD, "noop")
    with pytest.raises(RuntimeError, match="step failed"):
        control.agree("rank 0: boom", dist.group.WORLD, "step")
    with pytest.raises(RuntimeError, match="boom"):
        control.run_agreed(lambda: (_ for _ in ()).throw(ValueError("boom")), dist.group.WORLD, "step", 0)
    assert control.run_agreed(lambda: 7, dist.group.WORLD, "step", 0) == 7
