"""The progress watchdog reports stalled launches and does nothing else (no GPU needed: launches are stand-ins)."""

import time

import pytest

from pcie_ep_b200.utils.watchdog import ProgressWatchdog


def _wait_for(predicate, seconds=2.0):
    deadline = time.monotonic() + seconds
    while time.monotonic() < deadline:
        if predicate():
            return True
        time.sleep(0.01)
    return False


def test_reports_a_launch_that_does_not_finish_once_and_again_when_it_does():
    seen = []
    state = {"done": False}
    with ProgressWatchdog(limit_s=0.1, report=seen.append, poll_s=0.01) as dog:
        dog.watch("rank 0 launch 1", lambda: True)                 # finishes at once: never mentioned
        dog.watch("rank 0 launch 2", lambda: state["done"])
        assert _wait_for(lambda: len(seen) == 1)
        assert seen[0]["label"] == "rank 0 launch 2" and seen[0]["state"] == "still running" and seen[0]["waited_s"] > 0.1
        time.sleep(0.15)
        assert len(seen) == 1                                      # one report per stall, not one per poll
        assert dog.pending() == 1
        state["done"] = True
        assert _wait_for(lambda: len(seen) == 2)
        assert seen[1]["state"] == "finished late" and dog.pending() == 0
        assert [r["label"] for r in dog.reports] == ["rank 0 launch 2", "rank 0 launch 2"]


def test_a_failing_query_or_callback_never_stops_the_watchdog():
    def broken():
        raise RuntimeError("context is gone")

    def bad_callback(entry):
        raise ValueError("reporting failed")

    state = {"done": False}
    with ProgressWatchdog(limit_s=0.05, report=bad_callback, poll_s=0.01) as dog:
        dog.watch("a", broken)
        dog.watch("b", lambda: state["done"])
        assert _wait_for(lambda: any(r["state"].startswith("query failed") for r in dog.reports))
        assert _wait_for(lambda: any(r["label"] == "b" and r["state"] == "still running" for r in dog.reports))
    with pytest.raises(RuntimeError):
        dog.watch("c", lambda: True)                               # closed


def test_arguments_are_checked_and_the_default_report_goes_to_warnings():
    import warnings

    with pytest.raises(ValueError):
        ProgressWatchdog(limit_s=0)
    with pytest.raises(ValueError):
        ProgressWatchdog(limit_s=1.0, poll_s=0)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")                            # (raised in the watchdog's own thread)
        with ProgressWatchdog(limit_s=0.02, poll_s=0.005) as dog:
            dog.watch("stuck", lambda: False)
            assert _wait_for(lambda: len(dog.reports) == 1)
            assert dog.reports[0]["state"] == "still running"


def test_buffer_hands_every_launch_to_an_attached_watchdog():
    """The hook itself: the buffer's launch path registers the launch's event query under a label that names the rank."""
    import inspect

    from pcie_ep_b200.buffers import ep

    source = inspect.getsource(ep.HostStagedEPBuffer._enqueue)
    assert "self._watchdog.watch(" in source and "event.query" in source
    assert "attach_watchdog" in dir(ep.HostStagedEPBuffer)
