"""Stream-dependency wrapper handed out with every dispatch/combine result.

Same contract as the reference's ``EventOverlap`` (``pcie_ep/utils/event.py:10-100``):
waiting only enqueues a device-side dependency, the calling CPU thread never
blocks; a wait also tells the owning buffer which stream consumes the result so
that the result pool is not overwritten under a queued reader.

The class works with CUDA events and, for the CPU transport, with ``None``
events (a CPU result is complete when the call returns).
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch


class EventOverlap:
    """One completion dependency plus the objects queued GPU work still needs."""

    def __init__(
        self, event: Any = None, extra_tensors: Any = None, on_wait: Optional[Callable[[Any], None]] = None
    ) -> None:
        self.event = event
        self.extra_tensors = extra_tensors
        self._on_wait = on_wait
        self.hook_after_wait: Optional[Callable[[], Any]] = None
        self._release_handle_by_call = False
        self._released = False

    def current_stream_wait(self, release_handle: bool = False) -> Any:
        """Make the current stream wait for the event; return the hook's result once."""
        if self._released:
            raise RuntimeError("The event has already been released")
        if self.event is not None:
            stream = torch.cuda.current_stream()
            stream.wait_event(self.event)
            _record_tensors(self.extra_tensors, stream)
            if self._on_wait is not None:
                self._on_wait(stream)
        result = None
        if self.hook_after_wait is not None:
            hook, self.hook_after_wait = self.hook_after_wait, None
            result = hook()
        if release_handle:
            self.event = None
            self.extra_tensors = None
            self._on_wait = None
            self._released = True
        return result

    def wait(self) -> Any:
        return self.current_stream_wait()

    def register_hook_after_wait(self, hook_after_wait: Callable[[], Any]) -> None:
        if self.hook_after_wait is not None:
            raise RuntimeError("An epilogue hook is already registered")
        self.hook_after_wait = hook_after_wait

    def __call__(self, release_handle: bool = False) -> "EventOverlap":
        self._release_handle_by_call = release_handle
        return self

    def __enter__(self) -> "EventOverlap":
        return self

    def __exit__(self, exc_type: Any, exc_value: Any, traceback: Any) -> None:
        try:
            if not self._released:
                self.current_stream_wait(self._release_handle_by_call)
        finally:
            self._release_handle_by_call = False


def _record_tensors(value: Any, stream: Any) -> None:
    """``record_stream`` every CUDA tensor found in a nested container."""
    if isinstance(value, torch.Tensor):
        if value.is_cuda:
            value.record_stream(stream)
    elif isinstance(value, dict):
        for child in value.values():
            _record_tensors(child, stream)
    elif isinstance(value, (list, tuple)):
        for child in value:
            _record_tensors(child, stream)
