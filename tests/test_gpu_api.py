"""Public API on one real GPU rank (world size 1, in-process): cached layouts, CUDA-graph replay,
streams/events, pools, invalid routes, combine -- the reference's integration, cache/graph and
consumer-lifetime suites (tests/test_integration.py, tests/test_s6.py, tests/test_consumer_lifetime.py)
scaled to what one rank can show.  Multi-rank variants of the same kernels run in test_gpu_dispatch.py
(emulated ranks) and test_gpu_multiprocess.py (one process per GPU)."""

import tempfile

import pytest
import torch
import torch.distributed as dist

from pcie_ep_b200 import HostStagedConfig, HostStagedEPBuffer
from pcie_ep_b200.ops import reference
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu

EXPERTS, TOPK, HIDDEN, TMAX = 16, 4, 512, 64


@pytest.fixture(scope="module")
def world1():
    if not dist.is_initialized():
        store = dist.FileStore(tempfile.mktemp(prefix="gpu-api-store-"), 1)
        dist.init_process_group("gloo", store=store, rank=0, world_size=1)
    torch.cuda.set_device(0)
    yield


def _buffer(**kwargs):
    config = HostStagedConfig(channels=4, timeout_ms=3000, tx_warps=2, rx_warps=3, **kwargs)
    return HostStagedEPBuffer(None, TMAX, HIDDEN, TOPK, EXPERTS, config)


def _dev_inputs(tokens=TMAX, seed=7, pattern="random"):
    cpu = make_inputs(0, 1, tokens, HIDDEN, EXPERTS, TOPK, pattern, seed=seed)
    return cpu, tuple(t.cuda() for t in cpu)


def _check(result_tuple, cpu_inputs, expand, alignment=1, wire="bf16"):
    recv_x, recv_idx, recv_w, handle, event = result_tuple
    event.current_stream_wait()
    torch.cuda.synchronize()
    expected = reference.dispatch_reference([cpu_inputs], 0, EXPERTS, TMAX, do_expand=expand,
                                            expert_alignment=alignment, wire_dtype=wire)
    problems = reference.compare_dispatch(dict(handle._result), expected, do_expand=expand, do_zero_padding=False)
    assert not problems, problems


def test_cached_layout_repeats_and_detaches_from_pools(world1):
    with _buffer(output_pool_size=2) as buffer:
        cpu, (x, idx, w) = _dev_inputs()
        first = buffer.dispatch(x, idx, w, do_expand=True)
        _check(first, cpu, True)
        cache = buffer.cache_layout(first[3])
        del first
        for repeat in range(25):  # a cache never holds a result pool: 25 repeats with 2 pools
            x2 = (x.float() + repeat).to(torch.bfloat16)
            w2 = w * (1 + repeat)
            result = buffer.dispatch(x2, topk_weights=w2, handle=cache, do_expand=True)
            if repeat % 8 == 0:
                _check(result, (x2.cpu(), cpu[1], w2.cpu()), True)
            del result
        with pytest.raises(ValueError):
            buffer.dispatch(x, handle=cache, do_expand=False)
        buffer.check_errors()


def test_graph_replay_dynamic_and_cached(world1):
    with _buffer(enable_graph=True) as buffer:
        cpu, (x, idx, w) = _dev_inputs()
        graph = buffer.capture_dispatch(x, idx, w, do_expand=True)
        with pytest.raises(RuntimeError, match="one fixed-address"):
            buffer.capture_dispatch(x, idx, w, do_expand=True)
        for replay in range(5):
            # dynamic graph: payload, weights *and routes* may change in place between replays
            new_cpu = make_inputs(0, 1, TMAX, HIDDEN, EXPERTS, TOPK, "random", seed=50 + replay)
            x.copy_(new_cpu[0].cuda())
            idx.copy_(new_cpu[1].cuda())
            w.copy_(new_cpu[2].cuda())
            _check(graph.replay(), new_cpu, True)
            # eager dispatches interleave with replays
            _check(buffer.dispatch(x, idx, w, do_expand=False), new_cpu, False)
        with pytest.raises(ValueError, match="address"):
            graph.x = x.clone()
            graph.replay()
        buffer.check_errors()
    with _buffer(enable_graph=True) as buffer:
        cpu, (x, idx, w) = _dev_inputs(seed=3)
        cache = buffer.cache_layout(buffer.dispatch(x, idx, w, do_expand=True, expert_alignment=8)[3])
        graph = buffer.capture_dispatch(x, topk_weights=w, handle=cache, do_expand=True)
        assert graph.expert_alignment == 8
        for replay in range(3):
            x.mul_(0.5)
            _check(graph.replay(), (x.cpu(), cpu[1], cpu[2]), True, alignment=8)
        graph.close()
        with pytest.raises(RuntimeError):
            graph.replay()


def test_capture_requires_enable_graph(world1):
    with _buffer() as buffer:
        _, (x, idx, w) = _dev_inputs()
        with pytest.raises(NotImplementedError):
            buffer.capture_dispatch(x, idx, w)


def test_streams_previous_event_and_async(world1):
    with _buffer() as buffer:
        cpu, (x, idx, w) = _dev_inputs()
        assert buffer.get_comm_stream() != torch.cuda.current_stream()
        producer = torch.cuda.Stream()
        with torch.cuda.stream(producer):
            x2 = x * 2
            produced = HostStagedEPBuffer.capture()
        with pytest.raises(ValueError):
            buffer.dispatch(x2, idx, w, previous_event=produced)
        result = buffer.dispatch(x2, idx, w, do_expand=True, previous_event=produced, allocate_on_comm_stream=True,
                                 async_with_compute_stream=True)
        consumer = torch.cuda.Stream()
        with torch.cuda.stream(consumer):
            result[4].current_stream_wait()
            copy = result[0].clone()
        consumer.synchronize()
        assert (consumer.device.index, int(consumer.cuda_stream)) in buffer._consumer_streams
        _check(result, ((cpu[0] * 2), cpu[1], cpu[2]), True)
        expected = reference.dispatch_reference([((cpu[0] * 2), cpu[1], cpu[2])], 0, EXPERTS, TMAX, do_expand=True)
        rows = expected["valid_rows"]
        assert torch.equal(copy.cpu()[rows], expected["recv_x"][rows])
        # a raw torch event works as previous_event too
        raw = torch.cuda.Event()
        raw.record()
        _check(buffer.dispatch(x, idx, w, previous_event=raw, allocate_on_comm_stream=True), cpu, False)
        # deferred epilogue
        overlap = buffer.dispatch(x, idx, w, async_with_compute_stream=True, defer_epilogue=True)
        outputs = overlap.wait()
        assert len(outputs) == 4 and overlap.wait() is None
        buffer.check_errors()


def test_consumer_sees_original_data_after_references_dropped(world1):
    """A reader queued on its own stream must see its dispatch's rows even when the Python tensors are
    gone and later dispatches reuse the pool (reference: tests/test_consumer_lifetime.py)."""
    with _buffer(output_pool_size=2) as buffer:
        cpu, (x, idx, w) = _dev_inputs()
        result = buffer.dispatch(x, idx, w, do_expand=True, async_with_compute_stream=True)
        consumer = torch.cuda.Stream()
        with torch.cuda.stream(consumer):
            result[4].current_stream_wait()
            torch.cuda._sleep(20_000_000)  # the reader is slow
            snapshot = result[0].clone()
        del result
        for i in range(5):
            other = buffer.dispatch((x.float() + 100 + i).to(torch.bfloat16), idx, w, do_expand=True)
            del other
        torch.cuda.synchronize()
        expected = reference.dispatch_reference([cpu], 0, EXPERTS, TMAX, do_expand=True)
        rows = expected["valid_rows"]
        assert torch.equal(snapshot.cpu()[rows], expected["recv_x"][rows])


def test_cumulative_stats_and_invalid_routes(world1):
    with _buffer() as buffer:
        cpu, (x, idx, w) = _dev_inputs()
        totals = torch.zeros(EXPERTS, dtype=torch.int32, device="cuda")
        for _ in range(3):
            res = buffer.dispatch(x, idx, w, do_expand=True, cumulative_local_expert_recv_stats=totals)
            del res
        torch.cuda.synchronize()
        assert torch.equal(totals.cpu(), 3 * torch.bincount(cpu[1].flatten(), minlength=EXPERTS).to(torch.int32))
    for mutate in ("duplicate", "negative", "out_of_range"):
        with _buffer() as buffer:
            cpu, (x, idx, w) = _dev_inputs()
            bad = idx.clone()
            if mutate == "duplicate":
                bad[3, 1] = bad[3, 0]
            elif mutate == "negative":
                bad[3, 1] = -2
            else:
                bad[3, 1] = EXPERTS
            buffer.dispatch(x, bad, w, do_expand=True)
            with pytest.raises(RuntimeError, match=r"\[2, 3, 1"):
                buffer.check_errors()
            with pytest.raises(RuntimeError, match="failed"):
                buffer.dispatch(x, idx, w)


@pytest.mark.parametrize("mode", ["auto", "inline"])
def test_combine_weighted_and_unique(world1, mode):
    """Single rank: "auto" is the one-launch gather-reduce, "inline" the cooperative kernel writing straight to out."""
    with _buffer(combine_reduce=mode) as buffer:
        assert buffer.runtime.combine_is_local() == (mode == "auto")
        cpu, (x, idx, w) = _dev_inputs(pattern="partial")
        recv_x, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=True)
        combined, _, event = buffer.combine(recv_x, handle)
        event.current_stream_wait()
        want = cpu[0].float() * (cpu[2] * (cpu[1] >= 0)).sum(dim=1, keepdim=True)
        assert torch.allclose(combined.cpu().float(), want, rtol=2e-2, atol=2e-2)
        out = torch.empty_like(x)
        combined2, _, _ = buffer.combine(recv_x, handle, out=out, weighted=False)
        assert combined2.data_ptr() == out.data_ptr()
        want2 = cpu[0].float() * (cpu[1] >= 0).sum(dim=1, keepdim=True)
        torch.cuda.synchronize()
        assert torch.allclose(out.cpu().float(), want2, rtol=2e-2, atol=2e-2)
        del recv_x, handle, combined, combined2
        recv_x, _, _, handle, _ = buffer.dispatch(x, idx, w, do_expand=False)
        combined, _, _ = buffer.combine(recv_x, handle)
        torch.cuda.synchronize()
        hit = ((cpu[1] >= 0).any(dim=1, keepdim=True)).float()
        assert torch.allclose(combined.cpu().float(), cpu[0].float() * hit, rtol=1e-2, atol=1e-2)
        del recv_x, handle, combined
        # tokens that are routed nowhere come back as zero rows, also into a caller's dirty output tensor
        idx2 = idx.clone()
        idx2[::2] = -1
        recv_x, _, _, handle, _ = buffer.dispatch(x, idx2, w, do_expand=True)
        out = torch.full_like(x, 7.0)
        buffer.combine(recv_x, handle, out=out)
        torch.cuda.synchronize()
        want3 = cpu[0].float() * (cpu[2] * (idx2.cpu() >= 0)).sum(dim=1, keepdim=True)
        assert torch.allclose(out.cpu().float(), want3, rtol=2e-2, atol=2e-2)
        assert float(out[::2].abs().max()) == 0.0
        buffer.check_errors()


def test_large_and_small_buffers_alive_together(world1):
    """Two buffers with very different shared-memory needs share the kernels' opt-in attribute, which is only
    ever raised (reference: tests/test_f2_buffers.py): dispatches interleave and stay exact on both, whichever
    was built first, and closing one leaves the other working."""
    small_cfg = HostStagedConfig(channels=4, timeout_ms=3000, tx_warps=1, rx_warps=1)
    large_cfg = HostStagedConfig(channels=4, timeout_ms=3000, tx_warps=2, rx_warps=10)
    small = HostStagedEPBuffer(None, 32, 256, TOPK, EXPERTS, small_cfg)
    large = HostStagedEPBuffer(None, 32, 8192, TOPK, EXPERTS, large_cfg)
    assert large.runtime.shared_bytes() > small.runtime.shared_bytes()
    try:
        for step in range(6):
            for buffer, hidden in ((small, 256), (large, 8192)) if step % 2 else ((large, 8192), (small, 256)):
                cpu = make_inputs(0, 1, 32 - step, hidden, EXPERTS, TOPK, "random", seed=step)
                out = buffer.dispatch(*(t.cuda() for t in cpu), do_expand=True)
                out[4].current_stream_wait()
                torch.cuda.synchronize()
                expected = reference.dispatch_reference([cpu], 0, EXPERTS, 32, do_expand=True)
                assert not reference.compare_dispatch(dict(out[3]._result), expected, do_expand=True, do_zero_padding=False)
                del out
        large.close()
        cpu = make_inputs(0, 1, 32, 256, EXPERTS, TOPK, "random", seed=99)
        out = small.dispatch(*(t.cuda() for t in cpu), do_expand=True)
        torch.cuda.synchronize()
        expected = reference.dispatch_reference([cpu], 0, EXPERTS, 32, do_expand=True)
        assert not reference.compare_dispatch(dict(out[3]._result), expected, do_expand=True, do_zero_padding=False)
        del out
        small.check_errors()
    finally:
        small.close()
        large.close()
