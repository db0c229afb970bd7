"""Dispatch as a CUDA graph: captured once, collectively; replayed with no host work beyond the launch.

Parity: the reference's ``pcie_ep/graph.py:14-202`` (one graph per buffer, inputs bound by address, a
result pool of its own that the next replay overwrites, two agreement rounds around the capture).
The dispatch epoch lives on the device, so a replay carries no per-launch host state; every rank has
to replay in the same order, exactly as it has to call ``dispatch`` in the same order.
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Tuple

import torch

from .buffers import arguments
from .buffers.handle import HostStagedEPHandle
from .parallel import control
from .utils.event import EventOverlap, hold_for_stream


def _address_binding(tensor: Optional[torch.Tensor]) -> Optional[tuple]:
    """What a captured kernel argument depends on: where the tensor lives and how it is laid out."""
    if tensor is None:
        return None
    return (tensor.data_ptr(), tuple(tensor.shape), tuple(tensor.stride()), tensor.dtype, tensor.device)


class GraphDispatch:
    """One captured dispatch of one buffer.  Write new values *into* ``x`` / ``topk_idx`` /
    ``topk_weights`` (same tensors, same addresses), then ``replay()``.

    A graph captured with routing (``topk_idx`` given) recomputes the routing plan on every replay, so
    the routing tensor may change between replays.  A graph captured from a cached handle replays a
    fixed plan and refuses to run once that routing tensor has been written to.
    """

    def __init__(self, owner: Any, request: arguments.DispatchRequest, graph: Any, result: Any) -> None:
        self._owner = owner
        self._graph = graph
        self._result = result
        self._cache = request.source_handle
        self._born_in = owner._generation
        self._last_replay: Any = None
        self._open = True
        self.x, self.topk_idx, self.topk_weights = request.x, request.topk_idx, request.topk_weights
        self.do_expand, self.expert_alignment = request.expand, request.alignment
        self._captured_at = self._inputs_now()

    def _inputs_now(self) -> Tuple[Optional[tuple], ...]:
        return tuple(_address_binding(t) for t in (self.x, self.topk_idx, self.topk_weights))

    def _check_replayable(self) -> None:
        if not self._open or self._owner._generation != self._born_in:
            raise RuntimeError("this GraphDispatch was closed, or its buffer has been rebuilt since the capture")
        if self._inputs_now() != self._captured_at:
            raise ValueError("a captured dispatch reads fixed addresses: an input tensor's address, shape, dtype or stride changed")
        if self._cache is not None:
            self._cache.validate_cached(self._owner, self.x, self.expert_alignment, self.do_expand)

    def replay(self, *, previous_event: Any = None, async_with_compute_stream: bool = False) -> Any:
        """Enqueue the captured dispatch and return the usual five items.  No CPU wait, no read-back."""
        owner = self._owner
        with owner._lock:
            owner._check_live()
            self._check_replayable()
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("replay() launches a graph and cannot itself be captured")

            def launch(stream: Any) -> None:
                with torch.cuda.stream(stream):
                    self._graph.replay()

            _, event = owner._enqueue(launch, (), previous_event, async_with_compute_stream)
            self._last_replay = event
            keep = (owner, self, self.x, self.topk_idx, self.topk_weights, self._result)
            overlap = EventOverlap(event, keep, owner._register_consumer_stream)
            handle = HostStagedEPHandle(owner, self.topk_idx, self._result, self.do_expand, self.expert_alignment, overlap)
            owner._last_handle = handle
            weights = self._result.get("recv_topk_weights") if self.topk_weights is not None else None
            return self._result["recv_x"], self._result.get("recv_topk_idx"), weights, handle, overlap

    def close(self) -> None:
        """Wait for the last replay and free the graph.  The buffer's ``close`` does this as well."""
        if not self._open:
            return
        if self._last_replay is not None:
            self._last_replay.synchronize()
        self._graph.reset()
        self._open = False


def _agreed(step: Callable[[], Any], owner: Any, what: str, undo: Callable[[], None]) -> Any:
    """Run ``step`` on this rank, then let all ranks agree on whether it worked; ``undo`` runs if any rank failed."""
    value, problem = None, None
    try:
        value = step()
    except Exception as exc:  # noqa: BLE001 - reported to every rank below
        problem = f"rank {owner.rank_idx}: {type(exc).__name__}: {exc}"
    try:
        control.agree(problem, owner.control_group, what)
    except RuntimeError:
        undo()
        raise
    return value


def capture_dispatch(owner: Any, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None, *,
                     handle: Any = None, do_expand: bool = False, expert_alignment: Optional[int] = None,
                     do_zero_padding: bool = False) -> GraphDispatch:
    """Collective.  Validates, synchronises the device, captures one dispatch into the buffer's graph pool.

    Both phases end in an agreement round over the control group: a rank whose arguments are wrong, or
    whose capture fails, makes every rank raise instead of leaving the others inside a capture.
    """
    with owner._lock:
        owner._check_live()
        if not owner.on_gpu:
            raise NotImplementedError("capture_dispatch needs a GPU transport")
        if not owner.config.enable_graph:
            raise NotImplementedError("capture_dispatch needs a buffer built with enable_graph=True (it reserves the graph's result pool)")
        if owner._graph_capture is not None:
            raise RuntimeError("this buffer already holds its one fixed-address GraphDispatch; build a new buffer to capture again")

        holder = {}

        def prepare() -> arguments.DispatchRequest:
            request = arguments.build_dispatch_request(
                owner, x, topk_idx, topk_weights, handle=handle, expert_alignment=expert_alignment, do_expand=do_expand,
                do_zero_padding=do_zero_padding, alignment_limit=arguments.MAX_ALIGNMENT)
            torch.cuda.synchronize(owner.device)
            holder["graph"] = torch.cuda.CUDAGraph()
            return request

        def drop_graph() -> None:
            if "graph" in holder:
                holder["graph"].reset()

        request = _agreed(prepare, owner, "Collective graph preparation", drop_graph)
        graph = holder["graph"]
        comm = owner._streams.comm

        def capture() -> Any:
            hold_for_stream((request.x, request.topk_idx, request.topk_weights), comm)
            with torch.cuda.graph(graph, stream=comm):
                return owner.runtime.dispatch(request.x, request.topk_idx, request.topk_weights, request.alignment,
                                              request.expand, request.zero_padding, request.cached_layout, True)

        result = _agreed(capture, owner, "Collective graph capture", graph.reset)
        # a graph that recomputes its routing on every replay has no plan worth caching
        result["_layout"] = request.cached_layout
        captured = GraphDispatch(owner, request, graph, result)
        owner._graph_capture = captured
        return captured
