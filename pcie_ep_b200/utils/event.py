"""``EventOverlap``: the completion token that comes back with every dispatch and combine.

Parity: the reference's ``pcie_ep/utils/event.py:10-100`` (same public methods and the same one-shot
epilogue rule).  A token stands for device work that may still be running.  Waiting on it never blocks
the calling CPU thread: it lines the *current CUDA stream* up behind the work, pins the objects that
work still reads to that stream, and reports the stream to the owning buffer so that the buffer knows
who may still be reading a result pool.  Tokens of the CPU transport carry no event: their work was
complete when the call returned.
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch


def hold_for_stream(payload: Any, stream: Any) -> None:
    """Tell the caching allocator that ``stream`` uses every CUDA tensor inside ``payload``.

    ``payload`` may be a tensor or any nesting of lists, tuples and dicts; other objects are skipped.
    """
    pending = [payload]
    while pending:
        item = pending.pop()
        if isinstance(item, torch.Tensor):
            if item.is_cuda:
                item.record_stream(stream)
        elif isinstance(item, dict):
            pending.extend(item.values())
        elif isinstance(item, (list, tuple)):
            pending.extend(item)


class EventOverlap:
    """Completion of one piece of device work, plus what has to stay alive until it is consumed.

    ``event``          CUDA event recorded behind the work, or ``None`` (CPU transport).
    ``extra_tensors``  anything the queued work still references; kept alive by this object and pinned
                       to every stream that waits on it.
    ``on_wait``        callback ``f(stream)`` invoked with each waiting stream.
    """

    def __init__(self, event: Any = None, extra_tensors: Any = None,
                 on_wait: Optional[Callable[[Any], None]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors
        self._notify = on_wait
        self._epilogue: Optional[Callable[[], Any]] = None
        self._release_on_exit = False
        self._spent = False

    # -- waiting ---------------------------------------------------------------------------------
    def current_stream_wait(self, release_handle: bool = False) -> Any:
        """Order the current stream after the work.  The first wait returns the deferred epilogue's
        result (if one was registered), later waits return ``None``.  ``release_handle=True`` also drops
        the event and the pinned objects; the token cannot be waited on again afterwards."""
        if self._spent:
            raise RuntimeError("this EventOverlap has been released and can no longer be waited on")
        if self.event is not None:
            waiter = torch.cuda.current_stream()
            waiter.wait_event(self.event)
            hold_for_stream(self.extra_tensors, waiter)
            if self._notify is not None:
                self._notify(waiter)
        epilogue, self._epilogue = self._epilogue, None
        outcome = epilogue() if epilogue is not None else None
        if release_handle:
            self.event = self.extra_tensors = self._notify = None
            self._spent = True
        return outcome

    def wait(self) -> Any:
        return self.current_stream_wait()

    def register_hook_after_wait(self, hook_after_wait: Callable[[], Any]) -> None:
        """Attach the deferred epilogue; at most one may be pending."""
        if self._epilogue is not None:
            raise RuntimeError("an epilogue is already waiting on this EventOverlap")
        self._epilogue = hook_after_wait

    @property
    def hook_after_wait(self) -> Optional[Callable[[], Any]]:
        return self._epilogue

    # -- ``with event:`` / ``with event(release_handle=True):`` -----------------------------------
    def __call__(self, release_handle: bool = False) -> "EventOverlap":
        self._release_on_exit = bool(release_handle)
        return self

    def __enter__(self) -> "EventOverlap":
        return self

    def __exit__(self, exc_type: Any, exc_value: Any, traceback: Any) -> None:
        release, self._release_on_exit = self._release_on_exit, False
        if not self._spent:
            self.current_stream_wait(release)


# earlier name of the helper, still imported by user code
_record_tensors = hold_for_stream
