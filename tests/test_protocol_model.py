"""The host model of the dispatch and combine protocol: rules under ThreadSanitizer, failure scenarios on the CPU.

Ranks are threads over host memory with the kernels' own segment layout.  What the GPU suites may only do with
withheld flags and short timeouts -- and what they may not do at all, such as a rank that stops handing its
staging area back -- runs here with real concurrency and a race detector."""

import shutil

import pytest

from pcie_ep_b200.utils import protocol_model

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")

BASE = ["--ranks", 4, "--channels", 2, "--tokens", 48, "--slots", 2, "--hidden", 64]


def _tsan_works() -> bool:
    try:
        status, ranks, _ = protocol_model.run(["--ranks", 2, "--tokens", 8, "--epochs", 1], sanitize=True)
    except RuntimeError:
        return False
    return status == 0 and len(ranks) == 2


def test_epochs_with_bounded_rings_and_random_delays():
    status, ranks, _ = protocol_model.run(BASE + ["--epochs", 8, "--delay-us", 20])
    assert status == 0 and len(ranks) == 4
    assert all(r["error"] == 0 for r in ranks)
    # every row that was sent was received by someone, and the credit path was needed (more rows per ring than slots)
    assert sum(r["rows_sent"] for r in ranks) == sum(r["rows_received"] for r in ranks) > 4 * 8 * 48 / 2


@pytest.mark.parametrize("publish", ["release", "fenced"])
def test_both_correct_publication_chains_deliver_every_row(publish):
    status, ranks, _ = protocol_model.run(BASE + ["--epochs", 4, "--delay-us", 5, "--publish", publish, "--slots", 0])
    assert status == 0 and all(r["error"] == 0 for r in ranks)


def test_release_publication_is_race_free_under_thread_sanitizer():
    if not _tsan_works():
        pytest.skip("ThreadSanitizer is not usable with this compiler")
    status, ranks, stderr = protocol_model.run(BASE + ["--epochs", 4, "--delay-us", 10, "--publish", "release"], sanitize=True)
    assert "ThreadSanitizer" not in stderr, stderr[-1500:]
    assert status == 0 and all(r["error"] == 0 for r in ranks)


def test_a_relaxed_flag_without_a_fence_is_reported_as_a_race():
    """The chain that passed every two-GPU run and failed on four: the detector names it at once."""
    if not _tsan_works():
        pytest.skip("ThreadSanitizer is not usable with this compiler")
    status, _, stderr = protocol_model.run(BASE + ["--epochs", 2, "--delay-us", 10, "--publish", "relaxed"], sanitize=True)
    assert status != 0 and "data race" in stderr


@pytest.mark.parametrize("fault,code", [("--withhold-counts", 12), ("--skip-done", 11), ("--withhold-credit", 23), ("--corrupt-sequence", 18)])
def test_failure_scenarios_end_in_their_error_code_and_reach_every_rank(fault, code):
    status, ranks, _ = protocol_model.run(BASE + ["--epochs", 4, fault, 1, "--timeout-ms", 800, "--expect", code])
    assert status == 0, ranks
    codes = [r["error"] for r in ranks]
    assert code in codes                              # someone diagnosed the fault itself ...
    assert all(c in (code, 22) for c in codes if c)   # ... and everyone else who failed learned of it as a peer's abort
    if fault != "--corrupt-sequence":
        assert all(c != 0 for c in codes)             # a rank that goes silent stops every rank, within the timeout


def test_dispatch_followed_by_its_combine_every_epoch():
    status, ranks, _ = protocol_model.run(BASE + ["--combine", 1, "--epochs", 8, "--delay-us", 20])
    assert status == 0 and all(r["error"] == 0 for r in ranks)
    # an owner reads one landing row per (token, destination rank): exactly the rows it sent
    assert all(r["rows_combined"] == r["rows_sent"] > 0 for r in ranks)


def test_combine_is_race_free_under_thread_sanitizer():
    """Landing rows are plain stores and loads: the signal and the reuse guard are all that order them."""
    if not _tsan_works():
        pytest.skip("ThreadSanitizer is not usable with this compiler")
    status, ranks, stderr = protocol_model.run(BASE + ["--combine", 1, "--epochs", 4, "--delay-us", 10], sanitize=True)
    assert "ThreadSanitizer" not in stderr, stderr[-1500:]
    assert status == 0 and all(r["error"] == 0 and r["rows_combined"] == r["rows_sent"] for r in ranks)


@pytest.mark.parametrize("fault,code", [("--withhold-signal", 25), ("--skip-combine-done", 11)])
def test_combine_failure_scenarios(fault, code):
    """A rank that never says its combine rows are out stops the owners (signal wait); an owner that never hands its
    landing area back stops the next epoch's combine at the reuse guard."""
    status, ranks, _ = protocol_model.run(BASE + ["--combine", 1, "--epochs", 4, fault, 1, "--timeout-ms", 800, "--expect", code])
    assert status == 0, ranks
    codes = [r["error"] for r in ranks]
    assert code in codes and all(c in (code, 22) for c in codes) and all(codes)


@pytest.mark.parametrize("slots", [0, 2])
def test_the_cpu_relay_in_the_middle_forwards_every_remote_row(slots):
    """``--relay 1``: ranks write into outboxes, the product's ``NumaRelay`` (csrc/comm/numa_relay.hpp) forwards counts,
    rows, acknowledgements and hand-backs into the destinations' segments."""
    status, ranks, summary, _ = protocol_model.run_with_summary(BASE[:-4] + ["--slots", slots, "--hidden", 64, "--relay", 1, "--epochs", 6,
                                                                            "--delay-us", 20])
    assert status == 0 and all(r["error"] == 0 for r in ranks)
    assert sum(r["rows_sent"] for r in ranks) == sum(r["rows_received"] for r in ranks)
    assert summary["relay_failures"] == 0 and 0 < summary["relay_rows"] < sum(r["rows_sent"] for r in ranks)   # local rows bypass it


def test_the_cpu_relay_is_race_free_under_thread_sanitizer():
    """Product code under a race detector: the relay's worker threads against scripted senders and receivers."""
    if not _tsan_works():
        pytest.skip("ThreadSanitizer is not usable with this compiler")
    status, ranks, summary, stderr = protocol_model.run_with_summary(BASE + ["--relay", 1, "--epochs", 4, "--delay-us", 10], sanitize=True)
    assert "ThreadSanitizer" not in stderr, stderr[-1500:]
    assert status == 0 and all(r["error"] == 0 for r in ranks) and summary["relay_failures"] == 0


@pytest.mark.parametrize("fault,code", [("--withhold-counts", 12), ("--skip-done", 11), ("--withhold-credit", 23)])
def test_failures_reach_every_rank_through_the_relay(fault, code):
    """The abort flag is one of the things the relay forwards: a rank that goes silent still stops every rank."""
    status, ranks, summary, _ = protocol_model.run_with_summary(BASE + ["--relay", 1, "--epochs", 4, fault, 1, "--timeout-ms", 800,
                                                                        "--expect", code])
    assert status == 0, ranks
    codes = [r["error"] for r in ranks]
    assert code in codes and all(c in (code, 22) for c in codes) and all(codes) and summary["relay_failures"] == 0


def test_relay_and_combine_under_address_and_undefined_behaviour_sanitizers():
    try:
        protocol_model.build("address")
    except RuntimeError:
        pytest.skip("AddressSanitizer is not usable with this compiler")
    for extra in (["--relay", 1], ["--combine", 1]):
        status, ranks, stderr = protocol_model.run(BASE + extra + ["--epochs", 4, "--delay-us", 5], sanitize="address")
        assert "Sanitizer" not in stderr and "runtime error" not in stderr, stderr[-1500:]
        assert status == 0 and all(r["error"] == 0 for r in ranks)


@pytest.mark.parametrize("ranks,extra", [(8, ["--combine", 1, "--slots", 2]), (16, ["--relay", 1, "--slots", 0])])
def test_the_rank_counts_of_a_full_node_and_of_the_limit(ranks, extra):
    """Eight ranks (a node) with the combine, sixteen (the protocol's limit) through the relay: the segment layout's strides
    and the per-rank flag slots at the sizes the single-digit cases never reach."""
    status, ranks_out, _ = protocol_model.run(["--ranks", ranks, "--channels", 2, "--tokens", 32, "--hidden", 64, "--epochs", 3] + extra,
                                              timeout=300)
    assert status == 0 and len(ranks_out) == ranks and all(r["error"] == 0 for r in ranks_out)
    assert sum(r["rows_sent"] for r in ranks_out) == sum(r["rows_received"] for r in ranks_out) > 0


def test_the_relay_forwards_the_combine_rows_and_their_flags():
    """``--relay 1 --combine 1``: landing rows and their per-row flags (the one-kernel form of the combine, the one the relay
    serves) and the hand-back of the landing area all pass through the relay's threads -- also under ThreadSanitizer."""
    status, ranks, summary, _ = protocol_model.run_with_summary(BASE + ["--relay", 1, "--combine", 1, "--epochs", 5, "--delay-us", 10])
    assert status == 0 and all(r["error"] == 0 and r["rows_combined"] == r["rows_sent"] > 0 for r in ranks) and summary["relay_failures"] == 0
    if _tsan_works():
        status, ranks, _, stderr = protocol_model.run_with_summary(BASE + ["--relay", 1, "--combine", 1, "--epochs", 3, "--delay-us", 10],
                                                                   sanitize=True)
        assert "ThreadSanitizer" not in stderr, stderr[-1500:]
        assert status == 0 and all(r["error"] == 0 for r in ranks)


@pytest.mark.parametrize("fault,code", [("--withhold-signal", 15), ("--skip-combine-done", 11)])
def test_combine_failures_through_the_relay(fault, code):
    """Per-row flags that never come end the owners' row wait; a landing area never handed back ends the next reuse guard."""
    status, ranks, _, _ = protocol_model.run_with_summary(BASE + ["--relay", 1, "--combine", 1, "--epochs", 4, fault, 1, "--timeout-ms", 800,
                                                                  "--expect", code])
    assert status == 0, ranks
    codes = [r["error"] for r in ranks]
    assert code in codes and all(c in (code, 22) for c in codes) and all(codes)
