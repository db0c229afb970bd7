"""DeepEP-shaped expert-parallel buffer: ``dispatch`` and ``combine`` over peer HBM, host-staged
memory or a CPU (gloo) group.

The public surface -- constructor arguments, ``dispatch`` keywords, rejections, stream handling,
result pools, ``cache_layout``, ``capture_dispatch``, ``check_errors``, collective ``close`` -- is that
of the reference's ``HostStagedEPBuffer`` (``pcie_ep/buffers/ep.py:19-500``).  Differences:

* ``transport`` selects the substrate (``"peer"`` over NVLink by default on a GPU; ``"host_staged"``
  is the reference's substrate; ``"cpu"`` runs without a GPU);
* ``combine`` exists (the reference raises ``NotImplementedError``, ``ep.py:461-462``);
* one fused kernel launch per dispatch instead of eight.

Nothing on the dispatch/combine path waits on the CPU or issues a collective.
"""

from __future__ import annotations

import threading
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..config import HostStagedConfig
from ..parallel import control
from ..utils.event import EventOverlap, _record_tensors
from .handle import HostStagedEPHandle

_next_buffer_id = [0]


class _NullStream:
    """Stands in for a CUDA stream on the CPU transport: every operation is already ordered."""

    def wait_stream(self, other: Any) -> None:
        pass

    def wait_event(self, event: Any) -> None:
        pass


class HostStagedEPBuffer:
    """Collective owner of one EP communication context.

    Construction and ``close`` are collective over ``group`` and may block the CPU; ``dispatch`` and
    ``combine`` only enqueue device work.  CPU-side calls on one buffer must be serialised by the
    caller (a lock protects the internal bookkeeping, not the ordering of your launches).
    """

    def __init__(
        self,
        group: Any = None,
        num_max_tokens_per_rank: int = 0,
        hidden: int = 0,
        num_topk: int = 0,
        num_experts: int = 0,
        config: Optional[HostStagedConfig] = None,
        *,
        control_group: Any = None,
        host_staged_config: Optional[HostStagedConfig] = None,
        transport: Optional[str] = None,
        deterministic: bool = True,
        require_reuse_nccl_comm: bool = False,
        explicitly_destroy: bool = False,
    ) -> None:
        if not dist.is_initialized():
            raise RuntimeError("Initialize torch.distributed before constructing a buffer")
        if config is not None and host_staged_config is not None:
            raise ValueError("Supply config or host_staged_config, not both")
        self.config = config or host_staged_config or HostStagedConfig()
        if transport is not None and transport not in ("peer", "host_staged", "cpu", "auto"):
            raise ValueError("transport must be 'peer', 'host_staged', 'cpu' or 'auto'")
        chosen = transport if transport not in (None, "auto") else self.config.resolved_transport(torch.cuda.is_available())
        if chosen != "cpu" and not torch.cuda.is_available():
            raise RuntimeError(f"transport {chosen!r} requires NVIDIA CUDA")
        self.transport = chosen
        for name, value in (
            ("num_max_tokens_per_rank", num_max_tokens_per_rank),
            ("hidden", hidden),
            ("num_topk", num_topk),
            ("num_experts", num_experts),
        ):
            if not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be a positive integer")
        self.group = group if group is not None else dist.group.WORLD
        self.rank_idx = dist.get_rank(self.group)
        self.num_ranks = dist.get_world_size(self.group)
        if self.rank_idx < 0:
            raise ValueError("This process is not a member of the supplied EP group")
        self.global_ranks = tuple(dist.get_process_group_ranks(self.group))
        if num_experts % self.num_ranks:
            raise ValueError("Experts must be uniformly divisible among EP ranks")
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.hidden, self.num_topk, self.num_experts = hidden, num_topk, num_experts
        self.deterministic = deterministic
        self.explicitly_destroy = explicitly_destroy
        self.on_gpu = chosen != "cpu"
        self.device = torch.cuda.current_device() if self.on_gpu else "cpu"
        self._comm_stream = torch.cuda.Stream(device=self.device) if self.on_gpu else _NullStream()
        self._last_event = None
        self._last_handle: Optional[HostStagedEPHandle] = None
        self._generation = 0
        self._failed = False
        self._closed = False
        self._lock = threading.RLock()
        self._consumer_streams: Dict[tuple, Any] = {}
        self._graph_capture = None
        self._comm_busy = False  # work was queued on the communication stream that the compute stream has not waited for
        self._owns_control_group = False
        self.runtime = None
        self.segments = None
        self.relay = None
        self.directory = None
        self.nccl_comm = None
        self.comm_reused = False
        self.comm_reuse_status = "not_an_nccl_group"
        _next_buffer_id[0] += 1
        self.buffer_id = f"{self.rank_idx}-{_next_buffer_id[0]}"

        borrowed = control.borrow_nccl_comm(self.group, self.device, require_reuse=require_reuse_nccl_comm)
        self.nccl_comm, self.comm_reused, self.comm_reuse_status = borrowed.nccl_comm, borrowed.reused, borrowed.status

        self.control_group, self._owns_control_group = control.get_control_group(
            self.group, self.global_ranks, control_group
        )
        control.validate_group_configuration(
            self.control_group, self.num_ranks, num_max_tokens_per_rank, hidden, num_topk, num_experts,
            self.config, chosen,
        )
        options = self.config.native_options()
        if chosen == "cpu":
            from ..parallel.cpu_backend import CpuRuntime

            self.runtime = CpuRuntime(
                self.rank_idx, self.num_ranks, num_max_tokens_per_rank, hidden, num_topk, num_experts, options,
                self.control_group,
            )
            return

        # The extension is loaded (and built, if need be) only when a GPU buffer is constructed.
        from .. import _C
        from ..parallel.peer_memory import open_segments

        self._extension = _C
        layout = _C.segment_layout(
            self.num_ranks, self.config.channels, num_experts, num_topk, hidden, num_max_tokens_per_rank,
            self.config.payload_slots, self.config.enable_combine, self.config.fused_expert_combine,
        )
        self.segments = open_segments(
            _C, chosen, self.rank_idx, self.num_ranks, int(layout["size_bytes"]), self.device, self.control_group,
            self.config.directory, relay=self.config.numa_mode == "relay",
        )
        self.directory = self.segments.directory

        def make_runtime() -> Any:
            runtime = _C.Runtime(
                self.rank_idx, self.num_ranks, num_max_tokens_per_rank, hidden, num_topk, num_experts, options,
                self.segments.pointers, self.device,
            )
            # the dispatch stream must see fully initialised state without a CPU wait later on
            self._comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            return runtime

        self.runtime = control.run_agreed(make_runtime, self.control_group, "runtime construction", self.rank_idx)

        if self.config.numa_mode == "relay":
            def make_relay() -> Any:
                relay_options = {
                    "num_ranks": self.num_ranks, "channels": self.config.channels, "num_experts": num_experts,
                    "num_topk": num_topk, "hidden": hidden, "num_max_tokens": num_max_tokens_per_rank,
                    "payload_slots": self.config.payload_slots, "enable_combine": self.config.enable_combine,
                    "workers": self.config.relay_workers_per_numa, "cpu_affinity": list(self.config.relay_cpu_affinity),
                }
                relay = _C.NumaRelay(relay_options, self.segments.outbox_host_pointers, self.segments.host_pointers,
                                     self.rank_idx)
                relay.start()
                return relay

            self.relay = control.run_agreed(make_relay, self.control_group, "relay start", self.rank_idx)

    # ------------------------------------------------------------------ streams
    def get_comm_stream(self) -> Any:
        return self._comm_stream

    @staticmethod
    def _stream_key(stream: Any) -> tuple:
        return (stream.device.index, int(stream.cuda_stream))

    def _register_consumer_stream(self, stream: Any) -> None:
        """Remember a stream that reads results, even after the Python tensors are gone."""
        if not self.on_gpu:
            return
        with self._lock:
            key = self._stream_key(stream)
            if key != self._stream_key(self._comm_stream):
                self._consumer_streams[key] = stream

    def _wait_consumer_streams(self, compute: Any, compute_already_waited: bool) -> None:
        """Result pools are overwritten in place: order that after every registered reader's tail.

        Device-side waits only (reference: ``ep.py:204-220``).
        """
        if not self.on_gpu:
            return
        skip = {self._stream_key(self._comm_stream)}
        if compute_already_waited:
            skip.add(self._stream_key(compute))
        for key, stream in self._consumer_streams.items():
            if key not in skip:
                self._comm_stream.wait_stream(stream)
                skip.add(key)

    @staticmethod
    def capture() -> EventOverlap:
        """Record a producer dependency on the current CUDA stream."""
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream())
        return EventOverlap(event)

    def _current_stream(self) -> Any:
        return torch.cuda.current_stream(self.device) if self.on_gpu else _NullStream()

    def _launch_stream(self, compute: Any, previous_event: Any, async_with_compute_stream: bool) -> Any:
        """Pick the stream a launch goes to and set up its dependencies (device-side waits only).

        A synchronous call without a producer event is "communication stream waits for the compute
        stream, compute stream waits for the result": that is ordinary in-order execution, so the kernel
        is put on the compute stream itself and both cross-stream hand-offs (tens of microseconds of
        device latency per call) disappear.  Everything else goes to the communication stream.
        """
        if async_with_compute_stream or previous_event is not None:
            self._wait_for_inputs(compute, previous_event)
            self._comm_busy = True
            return self._comm_stream
        if self._comm_busy:
            compute.wait_stream(self._comm_stream)
            self._comm_busy = False
        skip = {self._stream_key(self._comm_stream), self._stream_key(compute)}
        for key, stream in self._consumer_streams.items():
            if key not in skip:
                compute.wait_stream(stream)
        return compute

    def _wait_for_inputs(self, compute: Any, previous_event: Any) -> None:
        if previous_event is None:
            self._comm_stream.wait_stream(compute)
        elif hasattr(previous_event, "current_stream_wait"):
            # an EventOverlap (or look-alike): the *communication* stream is the one that must wait
            if getattr(previous_event, "event", None) is not None:
                self._comm_stream.wait_event(previous_event.event)
            else:
                with torch.cuda.stream(self._comm_stream):
                    previous_event.current_stream_wait()
        else:
            self._comm_stream.wait_event(previous_event)
        self._wait_consumer_streams(compute, compute_already_waited=previous_event is None)

    # ------------------------------------------------------------------ dispatch
    def dispatch(
        self,
        x: torch.Tensor,
        topk_idx: Optional[torch.Tensor] = None,
        topk_weights: Optional[torch.Tensor] = None,
        cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
        num_experts: Optional[int] = None,
        num_max_tokens_per_rank: Optional[int] = None,
        expert_alignment: Optional[int] = None,
        num_sms: int = 0,
        num_qps: int = 0,
        previous_event: Any = None,
        async_with_compute_stream: bool = False,
        allocate_on_comm_stream: bool = False,
        handle: Any = None,
        do_handle_copy: bool = False,
        do_cpu_sync: Optional[bool] = False,
        do_expand: bool = False,
        do_zero_padding: bool = False,
        use_tma_aligned_col_major_sf: bool = False,
        defer_epilogue: bool = False,
    ) -> Any:
        """Send every token to the ranks that own its experts; sender and receiver deduplicated.

        ``x`` is contiguous BF16 ``[T, hidden]``, ``topk_idx`` int64 ``[T, K]`` of global expert ids
        (-1 = unused slot), ``topk_weights`` optional FP32 ``[T, K]``.  Returns
        ``(recv_x, recv_topk_idx, recv_topk_weights, handle, event)`` or, with ``defer_epilogue``, only
        the event whose first ``wait()`` returns the first four.  Shapes are capacities; the valid
        ranges are the device-side counts/offsets on the handle.  See the reference for the argument
        contract this follows (``pcie_ep/buffers/ep.py:229-360``).
        """
        with self._lock:
            self._check_live()
            if do_cpu_sync:
                raise NotImplementedError("The main path supports do_cpu_sync=False only")
            cached_layout = None
            if handle is not None:
                if topk_idx is not None:
                    raise ValueError("topk_idx must be None when a cached handle is supplied")
                topk_idx = handle.topk_idx
            if do_handle_copy or num_qps or num_sms or use_tma_aligned_col_major_sf:
                raise NotImplementedError("Handle copy, QPs, SM overrides and FP8 scale layouts are unsupported")
            if previous_event is not None and not allocate_on_comm_stream:
                raise ValueError("previous_event requires allocate_on_comm_stream=True")
            if defer_epilogue and not async_with_compute_stream:
                raise ValueError("defer_epilogue requires async_with_compute_stream=True")
            if do_zero_padding and not do_expand:
                raise ValueError("do_zero_padding is valid only with do_expand=True")
            alignment = (
                (handle.expert_alignment if handle is not None else 1) if expert_alignment is None else expert_alignment
            )
            if not isinstance(alignment, int) or isinstance(alignment, bool) or alignment < 1:
                raise ValueError("expert_alignment must be a positive integer")
            if num_experts not in (None, self.num_experts):
                raise ValueError("num_experts differs from the prepared buffer")
            if num_max_tokens_per_rank not in (None, self.num_max_tokens_per_rank):
                raise ValueError("num_max_tokens_per_rank differs from the prepared buffer")
            payload_dtype = torch.bfloat16 if self.on_gpu else None
            self._validate_input(x, "x", payload_dtype, (None, self.hidden))
            self._validate_input(topk_idx, "topk_idx", torch.int64, (x.shape[0], self.num_topk))
            if x.shape[0] > self.num_max_tokens_per_rank:
                raise ValueError("Input token count exceeds the prepared capacity")
            if topk_weights is not None:
                self._validate_input(topk_weights, "topk_weights", torch.float32, topk_idx.shape)
            if cumulative_local_expert_recv_stats is not None:
                self._validate_input(
                    cumulative_local_expert_recv_stats, "cumulative_local_expert_recv_stats", torch.int32,
                    (self.num_experts // self.num_ranks,),
                )
            if handle is not None:
                cached_layout = handle.validate_cached(self, x, alignment, do_expand)
            if self.on_gpu and torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("Use capture_dispatch for explicit CUDA Graph preparation")
            compute = self._current_stream()
            result, event = self._dispatch_on_comm_stream(
                x, topk_idx, topk_weights, cumulative_local_expert_recv_stats, alignment, do_expand,
                do_zero_padding, compute, previous_event, cached_layout, async_with_compute_stream,
            )
            refs = (self, x, topk_idx, topk_weights, result, cumulative_local_expert_recv_stats)
            if handle is not None:
                refs = (*refs, handle)
            overlap = EventOverlap(event, refs, self._register_consumer_stream)
            output_handle = HostStagedEPHandle(self, topk_idx, result, do_expand, alignment, overlap)
            self._last_event, self._last_handle = event, output_handle
            outputs = (
                result["recv_x"],
                result.get("recv_topk_idx"),
                result.get("recv_topk_weights") if topk_weights is not None else None,
                output_handle,
            )
            if not async_with_compute_stream and self.on_gpu:
                # result tensors live in pools owned by the runtime, not by the caching allocator:
                # nothing to record, but the reader stream must be known before the pool is reused
                if previous_event is not None:
                    compute.wait_event(event)
                    self._comm_busy = False
                self._register_consumer_stream(compute)
            if defer_epilogue:
                overlap.register_hook_after_wait(lambda: outputs)
                return overlap
            return (*outputs, overlap)

    def _dispatch_on_comm_stream(
        self, x, topk_idx, topk_weights, cumulative, alignment, do_expand, do_zero_padding, compute,
        previous_event, cached_layout=None, async_with_compute_stream=True,
    ):
        """Order dependencies, launch, record completion; never waits on the CPU."""
        if not self.on_gpu:
            result = self.runtime.dispatch(x, topk_idx, topk_weights, alignment, do_expand, do_zero_padding,
                                           cached_layout, False)
            if cumulative is not None:
                cumulative.add_(result["expert_counts"])
            return result, None
        comm = self._launch_stream(compute, previous_event, async_with_compute_stream)
        if comm is not compute:
            _record_tensors((x, topk_idx, topk_weights), comm)
        result = self.runtime.dispatch(x, topk_idx, topk_weights, alignment, do_expand, do_zero_padding,
                                       cached_layout, False, comm.cuda_stream)
        if cumulative is not None:
            with torch.cuda.stream(comm):
                cumulative.add_(result["expert_counts"])
                cumulative.record_stream(comm)
        event = torch.cuda.Event()
        event.record(comm)
        return result, event

    # ------------------------------------------------------------------ combine
    def combine(
        self,
        x: torch.Tensor,
        handle: HostStagedEPHandle,
        topk_weights: Optional[torch.Tensor] = None,
        *,
        out: Optional[torch.Tensor] = None,
        weighted: Optional[bool] = None,
        previous_event: Any = None,
        async_with_compute_stream: bool = False,
        allocate_on_comm_stream: bool = False,
    ) -> Any:
        """Return the expert outputs to their source tokens: the inverse of ``dispatch``.

        ``x`` holds this rank's expert outputs in the layout of the dispatch's ``recv_x``
        (expanded: one row per (token, local expert); unique: one row per token).  With the
        expanded layout each rank first reduces the rows of one source token with the weights that
        travelled with the dispatch (``weighted=False`` sums them unweighted), sends one BF16 row per
        (token, rank) back and the source adds the rows of all ranks in rank order in FP32.
        Returns ``(combined_x [T, hidden], None, event)``.
        """
        with self._lock:
            self._check_live()
            if topk_weights is not None:
                raise NotImplementedError("combine applies the weights given to dispatch; pass weighted=False to skip them")
            if not isinstance(handle, HostStagedEPHandle):
                raise TypeError("combine needs the handle returned by dispatch")
            if handle.buffer_id != self.buffer_id or handle.generation != self._generation:
                raise ValueError("The handle belongs to another buffer generation")
            if previous_event is not None and not allocate_on_comm_stream:
                raise ValueError("previous_event requires allocate_on_comm_stream=True")
            if weighted is None:
                weighted = handle.do_expand
            capacity = handle._result["recv_x"].shape[0]
            self._validate_input(x, "x", torch.bfloat16 if self.on_gpu else None, (None, self.hidden))
            if x.shape[0] > capacity:
                raise ValueError("combine input has more rows than the dispatch capacity")
            if not self.on_gpu:
                combined = self.runtime.combine(x, handle._result, weighted, out)
                return combined, None, EventOverlap(None, (self, x, handle, combined))
            if torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("combine cannot be issued inside a stream capture")
            compute = self._current_stream()
            comm = self._launch_stream(compute, previous_event, async_with_compute_stream)
            if comm is not compute:
                _record_tensors((x, out), comm)
            # without `out` the result is a preallocated pool tensor (busy while referenced)
            combined = self.runtime.combine(x, handle._result, weighted, out, comm.cuda_stream)
            event = torch.cuda.Event()
            event.record(comm)
            self._last_event = event
            overlap = EventOverlap(event, (self, x, handle, combined), self._register_consumer_stream)
            if not async_with_compute_stream:
                if previous_event is not None:
                    compute.wait_event(event)
                    self._comm_busy = False
                self._register_consumer_stream(compute)
            return combined, None, overlap

    def fused_expert_combine(self, hidden_rows: torch.Tensor, w_down: torch.Tensor, handle: HostStagedEPHandle,
                             *, out: Optional[torch.Tensor] = None) -> Any:
        """Down projection and combine in one pass: ``out[t] = sum_k w[t,k] * (hidden_rows[row(t,k)] @ w_down[e]^T)``.

        ``hidden_rows`` ``[rows, intermediate]`` are the expert activations in the layout of the (expanded)
        dispatch's ``recv_x``, ``w_down`` ``[local experts, hidden, intermediate]``.  The tcgen05 GEMM's epilogue
        multiplies every output row by the weight that travelled with the dispatch and stores it directly into
        the owner rank's landing slot ``(token, k)`` over NVLink while later tiles are still being multiplied; the
        owner then adds its K slots per token in slot order (FP32, deterministic).  Needs
        ``HostStagedConfig(fused_expert_combine=True)``.  Returns ``(combined_x [T, hidden], None, event)``.
        """
        with self._lock:
            self._check_live()
            if not self.config.fused_expert_combine:
                raise RuntimeError("this buffer was built with fused_expert_combine=False")
            if not isinstance(handle, HostStagedEPHandle):
                raise TypeError("fused_expert_combine needs the handle returned by dispatch")
            if handle.buffer_id != self.buffer_id or handle.generation != self._generation:
                raise ValueError("The handle belongs to another buffer generation")
            if not handle.do_expand:
                raise ValueError("fused_expert_combine needs a dispatch with do_expand=True")
            if not self.on_gpu:
                # CPU transport: the same result in two steps (matmul per expert, then the gloo combine)
                from ..ops.grouped_ffn import grouped_gemm

                rows = grouped_gemm(hidden_rows, w_down, handle.expert_offsets, handle.expert_counts, swiglu=False)
                combined = self.runtime.combine(rows, handle._result, True, out)
                return combined, None, EventOverlap(None, (self, hidden_rows, handle, combined))
            if torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("fused_expert_combine cannot be issued inside a stream capture")
            compute = self._current_stream()
            comm = self._launch_stream(compute, None, False)
            if comm is not compute:
                _record_tensors((hidden_rows, w_down, out), comm)
            self.runtime.fused_scatter_gemm(hidden_rows, w_down, handle._result, comm.cuda_stream)
            combined = self.runtime.fused_reduce(handle._result, out, comm.cuda_stream)
            event = torch.cuda.Event()
            event.record(comm)
            self._last_event = event
            self._register_consumer_stream(compute)
            return combined, None, EventOverlap(event, (self, hidden_rows, w_down, handle, combined), self._register_consumer_stream)

    # ------------------------------------------------------------------ cache / graph
    def capture_dispatch(self, *args: Any, **kwargs: Any) -> Any:
        """Collectively prepare the buffer's one fixed-address ``GraphDispatch``."""
        from ..graph import capture_dispatch

        return capture_dispatch(self, *args, **kwargs)

    def cache_layout(self, handle: HostStagedEPHandle) -> Any:
        """Detach the routing plan of ``handle`` without keeping its result pool busy."""
        self._check_live()
        if handle.buffer_id != self.buffer_id or handle.generation != self._generation:
            raise ValueError("The handle belongs to another buffer generation")
        return handle.cache_layout()

    # ------------------------------------------------------------------ validation / errors
    def _validate_input(self, tensor: Any, name: str, dtype: Any, shape: Any) -> None:
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch Tensor")
        if self.on_gpu:
            if not tensor.is_cuda or tensor.device.index != self.device:
                raise ValueError(f"{name} must be on this buffer's CUDA device")
        elif tensor.is_cuda:
            raise ValueError(f"{name} must be a CPU tensor for the cpu transport")
        if dtype is None:
            if not tensor.is_floating_point():
                raise ValueError(f"{name} must be a floating-point tensor")
        elif tensor.dtype != dtype:
            raise ValueError(f"{name} must be contiguous with dtype {dtype}")
        if not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous with dtype {dtype}")
        if tensor.ndim != len(shape) or any(
            expected is not None and actual != expected for actual, expected in zip(tensor.shape, shape)
        ):
            raise ValueError(f"{name} has shape {tuple(tensor.shape)}, expected {tuple(shape)}")

    def _check_live(self) -> None:
        if self._closed or self.runtime is None:
            raise RuntimeError("This buffer is closed")
        if self._failed:
            raise RuntimeError("This buffer has failed; do not dispatch again")
        if self.on_gpu and torch.cuda.current_device() != self.device:
            raise RuntimeError("The current CUDA device differs from the buffer's device")

    def check_errors(self, handle: Optional[HostStagedEPHandle] = None) -> None:
        """Explicit diagnostic: waits for the dispatch and reads its error words back."""
        selected = handle or self._last_handle
        if selected is None:
            return
        if selected.buffer_id != self.buffer_id or selected.generation != self._generation:
            raise ValueError("The handle belongs to a different buffer generation")
        if selected._completion_event is not None:
            selected._completion_event.synchronize()
        codes = selected.error.detach().cpu().reshape(-1).tolist()
        combine_error = selected._result.get("combine_error")
        if combine_error is not None:
            if self.on_gpu:
                torch.cuda.current_stream(self.device).synchronize()
                self._comm_stream.synchronize()
            codes_combine = combine_error.detach().cpu().reshape(-1).tolist()
            if any(codes_combine) and not any(codes):
                codes = codes_combine
        if any(codes):
            self._failed = True
            raise RuntimeError(f"EP dispatch GPU error on rank {self.rank_idx}: {codes}")

    # ------------------------------------------------------------------ close
    def close(self) -> None:
        """Collectively drain, release peer mappings, then free the segments."""
        with self._lock:
            if self._closed:
                return
            if self._graph_capture is not None:
                self._graph_capture.close()
                self._graph_capture = None
            if self.on_gpu:
                if self._last_event is not None:
                    self._last_event.synchronize()
                self._comm_stream.synchronize()
            dist.barrier(group=self.control_group)
            if self.relay is not None:
                self.relay.stop()
                self.relay = None
            self.runtime.close()
            self.runtime = None
            if self.segments is not None:
                self.segments.close(self.control_group, self._extension)
                self.segments = None
            else:
                dist.barrier(group=self.control_group)
            self._closed = True
            self._generation += 1
            self._last_handle = None
            self._consumer_streams.clear()
            if self._owns_control_group:
                dist.destroy_process_group(self.control_group)

    destroy = close

    def __enter__(self) -> "HostStagedEPBuffer":
        return self

    def __exit__(self, exc_type: Any, exc_value: Any, traceback: Any) -> None:
        self.close()


EPBuffer = HostStagedEPBuffer
