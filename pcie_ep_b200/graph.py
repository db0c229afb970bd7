"""Fixed-address CUDA-graph dispatch: capture once (collectively), then replay with no host work.

Same contract as the reference's ``GraphDispatch`` (``pcie_ep/graph.py:14-202``): one graph per buffer,
results in a dedicated pool that the next replay overwrites, inputs bound by address, the epoch lives
on the device so a replay needs nothing from the host, and both preparation steps end in an agreement
round so no rank is left alone inside a capture.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from .buffers.handle import HostStagedEPHandle
from .parallel import control
from .utils.event import EventOverlap, _record_tensors


def _signature(tensor: Any) -> Any:
    if tensor is None:
        return None
    return (tensor.data_ptr(), tuple(tensor.shape), tuple(tensor.stride()), tensor.dtype, tensor.device)


class GraphDispatch:
    """One captured dispatch bound to a buffer and to fixed input addresses."""

    def __init__(self, owner, x, topk_idx, weights, graph, result, alignment, expand, cached_handle) -> None:
        self._owner = owner
        self.x, self.topk_idx, self.topk_weights = x, topk_idx, weights
        self._graph, self._result = graph, result
        self.expert_alignment, self.do_expand = alignment, expand
        self._cached_handle = cached_handle
        self._bindings = tuple(_signature(value) for value in (x, topk_idx, weights))
        self._generation = owner._generation
        self._closed = False
        self._last_event = None

    def _validate_bindings(self) -> None:
        if self._closed or self._owner._generation != self._generation:
            raise RuntimeError("GraphDispatch is closed or its buffer generation changed")
        actual = tuple(_signature(value) for value in (self.x, self.topk_idx, self.topk_weights))
        if actual != self._bindings:
            raise ValueError("GraphDispatch input address, shape, dtype or strides changed")
        if self._cached_handle is not None:
            self._cached_handle.validate_cached(self._owner, self.x, self.expert_alignment, self.do_expand)

    def replay(self, *, previous_event: Any = None, async_with_compute_stream: bool = False) -> Any:
        """Enqueue the captured dispatch; returns the usual five items.  No CPU wait, no read-back."""
        owner = self._owner
        with owner._lock:
            owner._check_live()
            self._validate_bindings()
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("GraphDispatch.replay cannot be nested in another capture")
            compute = torch.cuda.current_stream(owner.device)
            stream = owner._launch_stream(compute, previous_event, async_with_compute_stream)
            with torch.cuda.stream(stream):
                self._graph.replay()
                event = torch.cuda.Event()
                event.record(stream)
            refs = (owner, self, self.x, self.topk_idx, self.topk_weights, self._result)
            overlap = EventOverlap(event, refs, owner._register_consumer_stream)
            handle = HostStagedEPHandle(owner, self.topk_idx, self._result, self.do_expand, self.expert_alignment, overlap)
            owner._last_event, owner._last_handle = event, handle
            self._last_event = event
            if not async_with_compute_stream:
                if previous_event is not None:
                    compute.wait_event(event)
                    owner._comm_busy = False
                owner._register_consumer_stream(compute)
            return (
                self._result["recv_x"],
                self._result.get("recv_topk_idx"),
                self._result.get("recv_topk_weights") if self.topk_weights is not None else None,
                handle,
                overlap,
            )

    def close(self) -> None:
        if self._closed:
            return
        if self._last_event is not None:
            self._last_event.synchronize()
        self._graph.reset()
        self._closed = True


def capture_dispatch(
    owner: Any,
    x: torch.Tensor,
    topk_idx: Optional[torch.Tensor] = None,
    topk_weights: Optional[torch.Tensor] = None,
    *,
    handle: Any = None,
    do_expand: bool = False,
    expert_alignment: Optional[int] = None,
    do_zero_padding: bool = False,
) -> GraphDispatch:
    """Collective.  May synchronise; the returned object's ``replay`` never does."""
    with owner._lock:
        owner._check_live()
        if not owner.on_gpu:
            raise NotImplementedError("capture_dispatch needs a GPU transport")
        if not owner.config.enable_graph:
            raise NotImplementedError("capture_dispatch requires enable_graph=True")
        if owner._graph_capture is not None:
            raise RuntimeError("A buffer supports one fixed-address GraphDispatch; rebuild it to recapture")
        graph, cached, alignment, error = None, None, None, None
        try:
            if handle is not None:
                if topk_idx is not None:
                    raise ValueError("topk_idx must be None when a cached handle is supplied")
                topk_idx = handle.topk_idx
            alignment = (handle.expert_alignment if handle is not None else 1) if expert_alignment is None else expert_alignment
            if not isinstance(alignment, int) or not 1 <= alignment <= 256:
                raise ValueError("expert_alignment must be in [1,256]")
            if do_zero_padding and not do_expand:
                raise ValueError("do_zero_padding requires do_expand=True")
            owner._validate_input(x, "x", torch.bfloat16, (None, owner.hidden))
            owner._validate_input(topk_idx, "topk_idx", torch.int64, (x.shape[0], owner.num_topk))
            if x.shape[0] > owner.num_max_tokens_per_rank:
                raise ValueError("Graph input exceeds the prepared capacity")
            if topk_weights is not None:
                owner._validate_input(topk_weights, "topk_weights", torch.float32, topk_idx.shape)
            if handle is not None:
                cached = handle.validate_cached(owner, x, alignment, do_expand)
            torch.cuda.synchronize(owner.device)
            graph = torch.cuda.CUDAGraph()
        except Exception as exc:  # noqa: BLE001 - agreed on below
            error = f"rank {owner.rank_idx}: {type(exc).__name__}: {exc}"
        try:
            control.agree(error, owner.control_group, "Collective graph preparation")
        except RuntimeError:
            if graph is not None:
                graph.reset()
            raise

        result, error = None, None
        try:
            with torch.cuda.stream(owner._comm_stream):
                _record_tensors((x, topk_idx, topk_weights), owner._comm_stream)
            with torch.cuda.graph(graph, stream=owner._comm_stream):
                result = owner.runtime.dispatch(x, topk_idx, topk_weights, alignment, do_expand, do_zero_padding, cached, True)
        except Exception as exc:  # noqa: BLE001
            error = f"rank {owner.rank_idx}: {type(exc).__name__}: {exc}"
        try:
            control.agree(error, owner.control_group, "Collective graph capture")
        except RuntimeError:
            graph.reset()
            raise
        # a dynamic graph recomputes its routing on every replay: its plan is not a cacheable layout
        result["_layout"] = cached
        captured = GraphDispatch(owner, x, topk_idx, topk_weights, graph, result, alignment, do_expand, handle)
        owner._graph_capture = captured
        return captured
