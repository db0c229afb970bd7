"""A host-side watchdog that reports launches which do not finish -- and does nothing else.

    watchdog = ProgressWatchdog(limit_s=5.0)
    buffer.attach_watchdog(watchdog)          # every dispatch / combine / fused launch is watched from now on
    ...
    for report in watchdog.reports: print(report)
    watchdog.close()

The kernels bound their own waits (``timeout_ms``) and leave with an error code, so a launch that never ends is not
expected; a peer process that died before launching its side, a full launch queue behind another stream, or a
misconfigured timeout are the cases a job wants to hear about while it is still running.  The watchdog only ever
*asks* whether an event has completed (a non-blocking query) and *reports* -- to a callback, to ``warnings`` and to
its ``reports`` list.  It never synchronises with, resets or otherwise touches a GPU context: on shared machines the
party that decides what to do about a stalled job is its owner, not a helper thread.
"""

from __future__ import annotations

import threading
import time
import warnings
from typing import Any, Callable, Dict, List, Optional


class ProgressWatchdog:
    def __init__(self, limit_s: float, report: Optional[Callable[[Dict[str, Any]], None]] = None, poll_s: float = 0.05) -> None:
        if limit_s <= 0 or poll_s <= 0:
            raise ValueError("limit_s and poll_s must be positive")
        self.limit_s = float(limit_s)
        self.poll_s = float(poll_s)
        self._report = report
        self._lock = threading.Lock()
        self._watched: List[Dict[str, Any]] = []
        self._reports: List[Dict[str, Any]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, name="ep-progress-watchdog", daemon=True)
        self._thread.start()

    def watch(self, label: str, is_done: Callable[[], bool]) -> None:
        """Watch one launch: ``is_done`` must be cheap and non-blocking (``torch.cuda.Event.query``)."""
        if self._stop.is_set():
            raise RuntimeError("the watchdog is closed")
        with self._lock:
            self._watched.append({"label": label, "is_done": is_done, "since": time.monotonic(), "reported": False})

    @property
    def reports(self) -> List[Dict[str, Any]]:
        with self._lock:
            return list(self._reports)

    def pending(self) -> int:
        with self._lock:
            return len(self._watched)

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=5.0)

    def __enter__(self) -> "ProgressWatchdog":
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()

    # ------------------------------------------------------------------ internals
    def _emit(self, entry: Dict[str, Any]) -> None:
        with self._lock:
            self._reports.append(entry)
        try:
            if self._report is not None:
                self._report(entry)
            else:
                warnings.warn(f"{entry['label']}: {entry['state']} after {entry['waited_s']:.1f} s", RuntimeWarning, stacklevel=2)
        except Exception:  # noqa: BLE001 - a reporting problem must never take the watchdog thread down
            pass

    def _loop(self) -> None:
        while not self._stop.wait(self.poll_s):
            now = time.monotonic()
            with self._lock:
                watched = list(self._watched)
            finished = []
            for item in watched:
                try:
                    done = bool(item["is_done"]())
                except Exception as exc:  # noqa: BLE001 - e.g. the context has gone; say so once and stop asking
                    self._emit({"label": item["label"], "state": f"query failed: {type(exc).__name__}", "waited_s": now - item["since"]})
                    finished.append(item)
                    continue
                if done:
                    if item["reported"]:
                        self._emit({"label": item["label"], "state": "finished late", "waited_s": now - item["since"]})
                    finished.append(item)
                elif not item["reported"] and now - item["since"] > self.limit_s:
                    item["reported"] = True
                    self._emit({"label": item["label"], "state": "still running", "waited_s": now - item["since"]})
            if finished:
                with self._lock:
                    self._watched = [w for w in self._watched if all(w is not f for f in finished)]
