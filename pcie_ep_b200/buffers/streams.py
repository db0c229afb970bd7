"""Stream policy of an EP buffer: which stream a launch goes to and what has to wait for what.

Result pools are overwritten in place, so the buffer must know every stream that may still be reading
an earlier result.  All dependencies set up here are device-side (``wait_stream`` / ``wait_event``);
nothing blocks the calling CPU thread.
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch


class NullStream:
    """Stands in for a CUDA stream on the CPU transport: every operation is already ordered."""

    cuda_stream = 0

    def wait_stream(self, other: Any) -> None:
        pass

    def wait_event(self, event: Any) -> None:
        pass

    def synchronize(self) -> None:
        pass


def stream_key(stream: Any) -> Tuple[int, int]:
    return (stream.device.index, int(stream.cuda_stream))


class StreamPolicy:
    """Owns the communication stream and the registry of consumer streams of one buffer.

    A *synchronous* call without a producer event means "the communication stream waits for the compute
    stream and the compute stream waits for the result", which is plain in-order execution: the kernel
    is put on the compute stream itself and both cross-stream hand-offs (tens of microseconds of device
    latency per call) disappear.  Asynchronous calls and calls with a producer event go to the
    communication stream.
    """

    def __init__(self, device: Any, on_gpu: bool) -> None:
        self.on_gpu = on_gpu
        self.device = device
        self.comm = torch.cuda.Stream(device=device) if on_gpu else NullStream()
        self.consumers: Dict[Tuple[int, int], Any] = {}
        # work was queued on the communication stream that the compute stream has not waited for yet
        self._comm_ahead = False

    def current(self) -> Any:
        return torch.cuda.current_stream(self.device) if self.on_gpu else NullStream()

    # -- readers of result pools ---------------------------------------------------------------
    def add_consumer(self, stream: Any) -> None:
        """Remember a stream that reads results; it outlives the Python tensors it reads."""
        if not self.on_gpu:
            return
        key = stream_key(stream)
        if key != stream_key(self.comm):
            self.consumers[key] = stream

    def _after_consumers(self, target: Any, *already_ordered: Any) -> None:
        """Make ``target`` wait for every registered reader except the streams given."""
        done = {stream_key(s) for s in already_ordered}
        done.add(stream_key(target))
        for key, reader in self.consumers.items():
            if key not in done:
                target.wait_stream(reader)

    # -- one launch ------------------------------------------------------------------------------
    def begin(self, compute: Any, previous_event: Any, run_async: bool) -> Any:
        """Return the stream the next kernel is launched on, with its input dependencies in place."""
        if not self.on_gpu:
            return compute
        if not run_async and previous_event is None:
            if self._comm_ahead:
                compute.wait_stream(self.comm)
                self._comm_ahead = False
            self._after_consumers(compute, self.comm)
            return compute
        if previous_event is None:
            self.comm.wait_stream(compute)
            self._after_consumers(self.comm, compute)
        else:
            self._wait_for_producer(previous_event)
            self._after_consumers(self.comm)
        self._comm_ahead = True
        return self.comm

    def _wait_for_producer(self, previous_event: Any) -> None:
        raw = getattr(previous_event, "event", None)
        if raw is not None:
            self.comm.wait_event(raw)  # an EventOverlap: the communication stream is the one that waits
        elif hasattr(previous_event, "current_stream_wait"):
            with torch.cuda.stream(self.comm):
                previous_event.current_stream_wait()
        else:
            self.comm.wait_event(previous_event)

    def finish(self, compute: Any, launched_on: Any, event: Optional[Any], run_async: bool) -> None:
        """After the launch of a synchronous call: the caller's stream sees the result and is recorded as a reader."""
        if not self.on_gpu or run_async:
            return
        if launched_on is not compute and event is not None:
            compute.wait_event(event)
            self._comm_ahead = False
        self.add_consumer(compute)

    def drain(self, last_event: Optional[Any]) -> None:
        """Blocking: used by ``close`` only."""
        if not self.on_gpu:
            return
        if last_event is not None:
            last_event.synchronize()
        self.comm.synchronize()
