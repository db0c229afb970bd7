"""DeepEP-shaped expert-parallel buffer: ``dispatch`` and ``combine`` over peer HBM, host-staged
memory or a CPU (gloo) group.

Parity: the reference's ``HostStagedEPBuffer`` (``pcie_ep/buffers/ep.py:19-500``) -- constructor
arguments, ``dispatch`` keywords and rejections, stream handling, result pools, ``cache_layout``,
``capture_dispatch``, ``check_errors``, collective ``close``.  Beyond it:

* ``transport`` selects the substrate (``"peer"`` over NVLink by default on a GPU, ``"host_staged"``
  over registered host memory, ``"cpu"`` without a GPU);
* ``combine`` and ``fused_expert_combine`` exist;
* a dispatch is one fused kernel launch.

Nothing on the dispatch/combine path waits on the CPU or issues a collective.
"""

from __future__ import annotations

import itertools
import threading
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..config import HostStagedConfig
from ..parallel import control
from ..utils.event import EventOverlap, hold_for_stream
from . import arguments
from .handle import HostStagedEPHandle
from .streams import StreamPolicy

_TRANSPORT_NAMES = ("peer", "host_staged", "cpu", "auto")
_buffer_serial = itertools.count(1)


class HostStagedEPBuffer:
    """Collective owner of one EP communication context.

    Construction and ``close`` are collective over ``group`` and may block the CPU; ``dispatch`` and
    ``combine`` only enqueue device work.  CPU-side calls on one buffer must be serialised by the
    caller (the internal lock protects bookkeeping, not the order of your launches).
    """

    def __init__(self, group: Any = None, num_max_tokens_per_rank: int = 0, hidden: int = 0, num_topk: int = 0, num_experts: int = 0,
                 config: Optional[HostStagedConfig] = None, *, control_group: Any = None,
                 host_staged_config: Optional[HostStagedConfig] = None, transport: Optional[str] = None, deterministic: bool = True,
                 require_reuse_nccl_comm: bool = False, explicitly_destroy: bool = False) -> None:
        if not dist.is_initialized():
            raise RuntimeError("Initialize torch.distributed (init_process_group) before building an EP buffer")
        if config is not None and host_staged_config is not None:
            raise ValueError("config and host_staged_config name the same thing: pass one of them, not both")
        self.config = config or host_staged_config or HostStagedConfig()
        if transport is not None and transport not in _TRANSPORT_NAMES:
            raise ValueError(f"unknown transport {transport!r}; choose from {_TRANSPORT_NAMES}")
        have_cuda = torch.cuda.is_available()
        chosen = self.config.resolved_transport(have_cuda) if transport in (None, "auto") else transport
        if chosen != "cpu" and not have_cuda:
            raise RuntimeError(f"transport {chosen!r} requires NVIDIA CUDA, which this process does not have")
        dims = dict(num_max_tokens_per_rank=num_max_tokens_per_rank, hidden=hidden, num_topk=num_topk, num_experts=num_experts)
        for name, value in dims.items():
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be a positive integer, got {value!r}")
        self.transport = chosen
        self.on_gpu = chosen != "cpu"
        self.group = dist.group.WORLD if group is None else group
        self.rank_idx = dist.get_rank(self.group)
        if self.rank_idx < 0:
            raise ValueError("the calling process is not part of the EP group it passed")
        self.num_ranks = dist.get_world_size(self.group)
        self.global_ranks = tuple(dist.get_process_group_ranks(self.group))
        if num_experts % self.num_ranks != 0:
            raise ValueError(f"{num_experts} experts cannot be split evenly over {self.num_ranks} ranks")
        self.num_max_tokens_per_rank, self.hidden = num_max_tokens_per_rank, hidden
        self.num_topk, self.num_experts = num_topk, num_experts
        self.deterministic, self.explicitly_destroy = deterministic, explicitly_destroy
        self.device = torch.cuda.current_device() if self.on_gpu else "cpu"
        self.buffer_id = f"{self.rank_idx}-{next(_buffer_serial)}"

        self._streams = StreamPolicy(self.device, self.on_gpu)
        self._lock = threading.RLock()
        self._generation = 0
        self._failed = self._closed = False
        self._last_event: Any = None
        self._watchdog: Any = None
        self._launches_watched = 0
        self._last_handle: Optional[HostStagedEPHandle] = None
        self._graph_capture: Any = None
        self._extension: Any = None
        self.runtime = self.segments = self.relay = self.directory = None

        borrowed = control.borrow_nccl_comm(self.group, self.device, require_reuse=require_reuse_nccl_comm)
        self.nccl_comm, self.comm_reused, self.comm_reuse_status = borrowed.nccl_comm, borrowed.reused, borrowed.status
        self.control_group, self._owns_control_group = control.get_control_group(self.group, self.global_ranks, control_group)
        control.validate_group_configuration(self.control_group, self.num_ranks, num_max_tokens_per_rank, hidden, num_topk,
                                             num_experts, self.config, chosen)
        if self.on_gpu:
            self._build_gpu_runtime()
        else:
            from ..parallel.cpu_backend import CpuRuntime

            self.runtime = CpuRuntime(self.rank_idx, self.num_ranks, num_max_tokens_per_rank, hidden, num_topk, num_experts,
                                      self.config.native_options(), self.control_group)

    def _build_gpu_runtime(self) -> None:
        """Segments, native runtime and (optionally) relay threads; every step ends in a collective agreement."""
        from .. import _C  # loaded (and built, if need be) only when a GPU buffer is constructed
        from ..parallel.peer_memory import open_segments

        self._extension = _C
        cfg = self.config
        layout = _C.segment_layout(self.num_ranks, cfg.channels, self.num_experts, self.num_topk, self.hidden,
                                   self.num_max_tokens_per_rank, cfg.payload_slots, cfg.enable_combine, cfg.fused_expert_combine)
        self.segments = open_segments(_C, self.transport, self.rank_idx, self.num_ranks, int(layout["size_bytes"]), self.device,
                                      self.control_group, cfg.directory, relay=cfg.numa_mode == "relay")
        self.directory = self.segments.directory

        options = cfg.native_options()
        options["segment_kind"] = self.transport  # where the segments live decides how flags are ordered after bulk copies

        def make_runtime() -> Any:
            runtime = _C.Runtime(self.rank_idx, self.num_ranks, self.num_max_tokens_per_rank, self.hidden, self.num_topk,
                                 self.num_experts, options, self.segments.pointers, self.device)
            # later launches on the communication stream must see fully initialised state without a CPU wait
            self._streams.comm.wait_stream(torch.cuda.current_stream(self.device))
            return runtime

        self.runtime = control.run_agreed(make_runtime, self.control_group, "runtime construction", self.rank_idx)
        if cfg.numa_mode != "relay":
            return

        # relay workers are grouped by the NUMA node of the destination GPU: every rank reports its own
        nodes = [None] * self.num_ranks
        dist.all_gather_object(nodes, int(_C.get_device_numa_node(self.device)), group=self.control_group)

        def make_relay() -> Any:
            options = dict(num_ranks=self.num_ranks, channels=cfg.channels, num_experts=self.num_experts,
                           target_numa_nodes=[max(0, n) for n in nodes],
                           num_topk=self.num_topk, hidden=self.hidden, num_max_tokens=self.num_max_tokens_per_rank,
                           payload_slots=cfg.payload_slots, enable_combine=cfg.enable_combine,
                           workers=cfg.relay_workers_per_numa, cpu_affinity=list(cfg.relay_cpu_affinity))
            relay = _C.NumaRelay(options, self.segments.outbox_host_pointers, self.segments.host_pointers, self.rank_idx)
            relay.start()
            return relay

        self.relay = control.run_agreed(make_relay, self.control_group, "relay start", self.rank_idx)

    # ------------------------------------------------------------------ streams
    def get_comm_stream(self) -> Any:
        return self._streams.comm

    @property
    def _comm_stream(self) -> Any:
        return self._streams.comm

    @property
    def _consumer_streams(self) -> dict:
        return self._streams.consumers

    def _register_consumer_stream(self, stream: Any) -> None:
        with self._lock:
            self._streams.add_consumer(stream)

    @staticmethod
    def capture() -> EventOverlap:
        """Record a producer dependency on the current CUDA stream (pass it as ``previous_event``)."""
        marker = torch.cuda.Event()
        marker.record(torch.cuda.current_stream())
        return EventOverlap(marker)

    def _enqueue(self, launch: Any, inputs: Any, previous_event: Any, run_async: bool) -> Any:
        """Run ``launch(stream_handle)`` on the stream the policy picks; returns (value, event, stream)."""
        compute = self._streams.current()
        stream = self._streams.begin(compute, previous_event, run_async)
        if stream is not compute:
            hold_for_stream(inputs, stream)
        value = launch(stream)
        event = torch.cuda.Event()
        event.record(stream)
        self._last_event = event
        self._streams.finish(compute, stream, event, run_async)
        if self._watchdog is not None:
            self._launches_watched += 1
            self._watchdog.watch(f"rank {self.rank_idx} launch {self._launches_watched}", event.query)
        return value, event

    def attach_watchdog(self, watchdog: Any) -> None:
        """Have ``watchdog`` (``pcie_ep_b200.utils.watchdog.ProgressWatchdog``, or None to detach) told about every
        launch of this buffer; it only queries the launch's event and reports, it never touches the GPU."""
        self._watchdog = watchdog

    # ------------------------------------------------------------------ dispatch
    def dispatch(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                 cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None, num_experts: Optional[int] = None,
                 num_max_tokens_per_rank: Optional[int] = None, expert_alignment: Optional[int] = None, num_sms: int = 0, num_qps: int = 0,
                 previous_event: Any = None, async_with_compute_stream: bool = False, allocate_on_comm_stream: bool = False,
                 handle: Any = None, do_handle_copy: bool = False, do_cpu_sync: Optional[bool] = False, do_expand: bool = False,
                 do_zero_padding: bool = False, use_tma_aligned_col_major_sf: bool = False, defer_epilogue: bool = False) -> Any:
        """Send every token to the ranks that own its experts; sender and receiver deduplicated.

        ``x`` is contiguous BF16 ``[T, hidden]``, ``topk_idx`` int64 ``[T, K]`` of global expert ids
        (-1 = unused slot), ``topk_weights`` optional FP32 ``[T, K]``.  Returns
        ``(recv_x, recv_topk_idx, recv_topk_weights, handle, event)`` or, with ``defer_epilogue``, only
        the event whose first ``wait()`` returns the first four.  Shapes are capacities; the valid
        ranges are the device-side counts and offsets on the handle.
        """
        with self._lock:
            self._check_live()
            arguments.reject_unsupported(dict(do_cpu_sync=do_cpu_sync, do_handle_copy=do_handle_copy, num_qps=num_qps,
                                              num_sms=num_sms, use_tma_aligned_col_major_sf=use_tma_aligned_col_major_sf))
            self._check_stream_options(previous_event, allocate_on_comm_stream)
            if defer_epilogue and not async_with_compute_stream:
                raise ValueError("defer_epilogue hands the outputs over at the first wait(), which needs async_with_compute_stream=True")
            request = arguments.build_dispatch_request(
                self, x, topk_idx, topk_weights, handle=handle, expert_alignment=expert_alignment, do_expand=do_expand,
                do_zero_padding=do_zero_padding, cumulative=cumulative_local_expert_recv_stats, num_experts=num_experts,
                num_max_tokens_per_rank=num_max_tokens_per_rank)
            if self.on_gpu and torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("dispatch cannot run inside a stream capture; capture_dispatch prepares a CUDA graph")
            result, event = self._launch_dispatch(request, previous_event, async_with_compute_stream)
            overlap = EventOverlap(event, request.keepalive(self, result), self._register_consumer_stream)
            out_handle = HostStagedEPHandle(self, request.topk_idx, result, request.expand, request.alignment, overlap)
            self._last_handle = out_handle
            outputs = (result["recv_x"], result.get("recv_topk_idx"),
                       result.get("recv_topk_weights") if request.topk_weights is not None else None, out_handle)
            if defer_epilogue:
                overlap.register_hook_after_wait(lambda: outputs)
                return overlap
            return (*outputs, overlap)

    def _launch_dispatch(self, request: arguments.DispatchRequest, previous_event: Any, run_async: bool) -> Any:
        """Order dependencies, launch, record completion; never waits on the CPU."""
        r = request
        if not self.on_gpu:
            result = self.runtime.dispatch(r.x, r.topk_idx, r.topk_weights, r.alignment, r.expand, r.zero_padding,
                                           r.cached_layout, False)
            if r.cumulative is not None:
                r.cumulative.add_(result["expert_counts"])
            return result, None

        def launch(stream: Any) -> Any:
            result = self.runtime.dispatch(r.x, r.topk_idx, r.topk_weights, r.alignment, r.expand, r.zero_padding,
                                           r.cached_layout, False, stream.cuda_stream)
            if r.cumulative is not None:
                with torch.cuda.stream(stream):
                    r.cumulative.add_(result["expert_counts"])
                    r.cumulative.record_stream(stream)
            return result

        return self._enqueue(launch, (r.x, r.topk_idx, r.topk_weights), previous_event, run_async)

    @staticmethod
    def _check_stream_options(previous_event: Any, allocate_on_comm_stream: bool) -> None:
        if previous_event is not None and not allocate_on_comm_stream:
            raise ValueError("previous_event moves the launch to the communication stream: pass allocate_on_comm_stream=True with it")

    def _check_handle(self, handle: Any, purpose: str) -> None:
        if not isinstance(handle, HostStagedEPHandle):
            raise TypeError(f"{purpose} takes the handle that dispatch returned, not {type(handle).__name__}")
        if (handle.buffer_id, handle.generation) != (self.buffer_id, self._generation):
            raise ValueError(f"{purpose}: the handle comes from another buffer, or from before this buffer was rebuilt")

    # ------------------------------------------------------------------ combine
    def combine(self, x: torch.Tensor, handle: HostStagedEPHandle, topk_weights: Optional[torch.Tensor] = None, *,
                out: Optional[torch.Tensor] = None, weighted: Optional[bool] = None, previous_event: Any = None,
                async_with_compute_stream: bool = False, allocate_on_comm_stream: bool = False, num_sms: int = 0) -> Any:
        """Return the expert outputs to their source tokens: the inverse of ``dispatch``.

        ``x`` holds this rank's expert outputs in the layout of the dispatch's ``recv_x``
        (expanded: one row per (token, local expert); unique: one row per token).  With the
        expanded layout each rank first reduces the rows of one source token with the weights that
        travelled with the dispatch (``weighted=False`` sums them unweighted), sends one BF16 row per
        (token, rank) back and the source adds the rows of all ranks in rank order in FP32.
        ``num_sms`` > 0 limits the two combine launches to that many SMs' worth of CTAs, so that an
        expert GEMM on another stream keeps the rest.  Returns ``(combined_x [T, hidden], None, event)``.
        """
        with self._lock:
            self._check_live()
            if topk_weights is not None:
                raise NotImplementedError("combine applies the weights that travelled with the dispatch; use weighted=False for a plain sum")
            self._check_handle(handle, "combine")
            self._check_stream_options(previous_event, allocate_on_comm_stream)
            if isinstance(num_sms, bool) or not isinstance(num_sms, int) or num_sms < 0:
                raise ValueError("num_sms must be a non-negative integer")
            use_weights = handle.do_expand if weighted is None else bool(weighted)
            arguments.TensorRule("x", torch.bfloat16 if self.on_gpu else None, (None, self.hidden)).check(
                x, device=self.device, on_gpu=self.on_gpu)
            capacity = handle._result["recv_x"].shape[0]
            if x.shape[0] > capacity:
                raise ValueError(f"x has {x.shape[0]} rows, the dispatch result holds at most {capacity}")
            if not self.on_gpu:
                combined = self.runtime.combine(x, handle._result, use_weights, out)
                return combined, None, EventOverlap(None, (self, x, handle, combined))
            if torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("combine cannot run inside a stream capture")
            # without `out` the result is a preallocated pool tensor (busy while referenced)
            combined, event = self._enqueue(
                lambda stream: self.runtime.combine(x, handle._result, use_weights, out, stream.cuda_stream, num_sms),
                (x, out), previous_event, async_with_compute_stream)
            return combined, None, EventOverlap(event, (self, x, handle, combined), self._register_consumer_stream)

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
            self._check_handle(handle, "fused_expert_combine")
            if not handle.do_expand:
                raise ValueError("fused_expert_combine works on the expanded layout: dispatch with do_expand=True")
            if not self.on_gpu:
                # CPU transport: the same result in two steps (matmul per expert, then the gloo combine)
                from ..ops.grouped_ffn import grouped_gemm

                rows = grouped_gemm(hidden_rows, w_down, handle.expert_offsets, handle.expert_counts, swiglu=False)
                combined = self.runtime.combine(rows, handle._result, True, out)
                return combined, None, EventOverlap(None, (self, hidden_rows, handle, combined))
            if torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("fused_expert_combine cannot run inside a stream capture")

            def launch(stream: Any) -> Any:
                self.runtime.fused_scatter_gemm(hidden_rows, w_down, handle._result, stream.cuda_stream)
                return self.runtime.fused_reduce(handle._result, out, stream.cuda_stream)

            combined, event = self._enqueue(launch, (hidden_rows, w_down, out), None, False)
            return combined, None, EventOverlap(event, (self, hidden_rows, w_down, handle, combined), self._register_consumer_stream)

    # ------------------------------------------------------------------ cache / graph
    def capture_dispatch(self, *args: Any, **kwargs: Any) -> Any:
        """Collectively prepare the buffer's one fixed-address ``GraphDispatch``."""
        from ..graph import capture_dispatch

        return capture_dispatch(self, *args, **kwargs)

    def cache_layout(self, handle: HostStagedEPHandle) -> Any:
        """Detach the routing plan of ``handle`` without keeping its result pool busy."""
        self._check_live()
        self._check_handle(handle, "cache_layout")
        return handle.cache_layout()

    # ------------------------------------------------------------------ state / errors
    def _check_live(self) -> None:
        if self._closed or self.runtime is None:
            raise RuntimeError("this EP buffer is closed")
        if self._failed:
            raise RuntimeError("this EP buffer has failed (see check_errors); close it and build a new one")
        if self.on_gpu and torch.cuda.current_device() != self.device:
            raise RuntimeError(f"the buffer lives on cuda:{self.device}, the current device is cuda:{torch.cuda.current_device()}")

    def check_errors(self, handle: Optional[HostStagedEPHandle] = None) -> None:
        """Explicit diagnostic: waits for the dispatch (and a combine issued after it) and raises on a device error."""
        target = handle if handle is not None else self._last_handle
        if target is None:
            return
        if (target.buffer_id, target.generation) != (self.buffer_id, self._generation):
            raise ValueError("check_errors: the handle comes from another buffer, or from before this buffer was rebuilt")
        if target._completion_event is not None:
            target._completion_event.synchronize()
        words = target.error.detach().cpu().reshape(-1).tolist()
        combine_words = target._result.get("combine_error")
        if combine_words is not None and not any(words):
            if self.on_gpu:
                torch.cuda.current_stream(self.device).synchronize()
                self._streams.comm.synchronize()
            words = combine_words.detach().cpu().reshape(-1).tolist()
        if any(words):
            self._failed = True
            raise RuntimeError(f"EP dispatch GPU error on rank {self.rank_idx}: {words}")

    # ------------------------------------------------------------------ close
    def close(self) -> None:
        """Collective: drain the streams, stop the relay, release peer mappings, free the segments."""
        with self._lock:
            if self._closed:
                return
            if self._graph_capture is not None:
                self._graph_capture.close()
                self._graph_capture = None
            self._streams.drain(self._last_event)
            dist.barrier(group=self.control_group)  # no rank unmaps while a peer's kernel may still write here
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
            self._streams.consumers.clear()
            if self._owns_control_group:
                dist.destroy_process_group(self.control_group)

    destroy = close

    def __enter__(self) -> "HostStagedEPBuffer":
        return self

    def __exit__(self, exc_type: Any, exc_value: Any, traceback: Any) -> None:
        self.close()


EPBuffer = HostStagedEPBuffer
