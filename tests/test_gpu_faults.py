"""Failure detection and protocol-ordering tests on emulated ranks (one GPU, one cooperative launch).

No test here faults, traps or hangs the GPU: failures are *withheld flags* (written, or rather not
written, by their legal owner through the runtime's test hooks) and every device wait gives up after
the configured timeout with an error code that the host reads afterwards.  Coverage follows the
reference's control-plane and ordering suites (tests/test_control_progress.py: prefix_timeout,
mailbox_timeout; tests/test_timeout.py: sticky failure; tests/test_protocol_stages.py and
tests/test_prefix_tx.py: injected delays, prefix/TX overlap)."""

import pytest
import torch

from pcie_ep_b200 import HostStagedConfig
from pcie_ep_b200.ops import reference
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu

WORLD, EXPERTS, TOPK, HIDDEN, TMAX = 4, 16, 4, 256, 32


def _group(timeout_ms=300, **kwargs):
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    config = HostStagedConfig(channels=2, timeout_ms=timeout_ms, tx_warps=2, rx_warps=2, **kwargs)
    return VirtualEPGroup(WORLD, TMAX, HIDDEN, TOPK, EXPERTS, config)


def _inputs(seed=7):
    cpu = [make_inputs(r, WORLD, TMAX, HIDDEN, EXPERTS, TOPK, "random", seed=seed) for r in range(WORLD)]
    dev = [tuple(t.cuda() for t in inp) for inp in cpu]
    return cpu, ([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev])


def _codes(results):
    torch.cuda.synchronize()
    return [r["error"].cpu().tolist() for r in results]


def test_withheld_counts_time_out_and_failure_is_sticky(ext):
    with _group(timeout_ms=200) as group:
        cpu, args = _inputs()
        ok = group.dispatch(*args, do_expand=True)
        assert all(code[0] == 0 for code in _codes(ok))
        del ok
        group.runtimes[2].set_test_withhold_counts(True)  # rank 2 never tells anybody what to expect
        failed = group.dispatch(*args, do_expand=True)
        codes = _codes(failed)
        # every rank ends with an error: its own counts wait (12) on source 2, or a peer's abort (22)
        assert all(code[0] in (12, 22) for code in codes), codes
        assert any(code[0] == 12 and code[1] == 2 for code in codes), codes
        del failed
        group.runtimes[2].set_test_withhold_counts(False)
        again = group.dispatch(*args, do_expand=True)  # terminal: the next launch refuses to run
        assert all(code[0] == 19 for code in _codes(again)), _codes(again)
        assert all(int(rt.sticky_error()[0]) != 0 for rt in group.runtimes)


def test_missing_done_flag_times_out_next_epoch(ext):
    """A rank that never hands its staging area back blocks the *next* epoch's reuse guard (error 11)."""
    with _group(timeout_ms=200) as group:
        cpu, args = _inputs()
        group.runtimes[0].set_test_skip_counts_ack_source(1)  # rank 0 will not publish `done` to rank 1
        first = group.dispatch(*args, do_expand=True)
        assert all(code[0] == 0 for code in _codes(first))
        del first
        second = group.dispatch(*args, do_expand=True)
        codes = _codes(second)
        assert codes[1][0] == 11 and codes[1][1] == 0, codes  # rank 1 waited for rank 0
        assert all(code[0] in (11, 12, 15, 22) for code in codes), codes


@pytest.mark.parametrize("which", ["metadata", "tx", "rx", "scatter"])
def test_injected_delays_keep_results_exact(ext, which):
    with _group(timeout_ms=2000) as group:
        delays = {"metadata": (100_000, 0, 0, 0), "tx": (0, 100_000, 0, 0), "rx": (0, 0, 100_000, 0),
                  "scatter": (0, 0, 0, 100_000)}[which]
        group.runtimes[WORLD - 1].set_test_delays(*delays)
        for epoch in range(3):
            cpu, args = _inputs(seed=30 + epoch)
            results = group.dispatch(*args, do_expand=True)
            torch.cuda.synchronize()
            for rank in range(WORLD):
                expected = reference.dispatch_reference(cpu, rank, EXPERTS, TMAX, do_expand=True)
                assert not reference.compare_dispatch(results[rank], expected, do_expand=True, do_zero_padding=False)
            del results


def test_sends_overlap_a_slow_receive_prefix(ext):
    """With the receive prefix delayed by 20 ms the sends still go out first (reference:
    tests/test_prefix_tx.py asserts prefix_start < first_payload_done < prefix_end)."""
    with _group(timeout_ms=2000) as group:
        for rt in group.runtimes:
            rt.set_test_prefix_delay_ns(20_000_000)
        cpu, args = _inputs()
        results = group.dispatch(*args, do_expand=True)
        torch.cuda.synchronize()
        for rank in range(WORLD):
            expected = reference.dispatch_reference(cpu, rank, EXPERTS, TMAX, do_expand=True)
            assert not reference.compare_dispatch(results[rank], expected, do_expand=True, do_zero_padding=False)
            stamps = results[rank]["prefix_tx_timestamps_ns"].cpu()
            prefix_start, prefix_end = int(stamps[0, 0]), int(stamps[0, 1])
            tx_done = [int(v) for v in stamps[1:, 1].tolist() if v > 0]
            assert prefix_end - prefix_start >= 20_000_000
            assert tx_done and max(tx_done) < prefix_end, "sends waited for the prefix"
            assert int(results[rank]["stats"][3]) > 0  # rows pushed before the prefix was ready
        # the next epochs start from clean READY state
        for rt in group.runtimes:
            rt.set_test_prefix_delay_ns(0)
        del results
        for epoch in range(2):
            cpu, args = _inputs(seed=60 + epoch)
            results = group.dispatch(*args, do_expand=True)
            assert all(code[0] == 0 for code in _codes(results))
            del results


def test_profiling_timestamps_are_monotonic(ext):
    with _group(timeout_ms=2000) as group:
        cpu, args = _inputs()
        results = group.dispatch(*args, do_expand=True)
        torch.cuda.synchronize()
        prof = results[0]["profiling"].cpu()
        start, split, end = prof[:, 0], prof[:, 7], prof[:, 14]
        assert (start > 0).all() and (split >= start).all() and (end >= split).all()


def test_row_with_wrong_sequence_is_refused(ext):
    """A row whose sequence words do not match the epoch of its READY flag ends the launch with error 18.

    The wrong sequence is written by the legal owner of the row (the sending rank's own send warps, through a
    test hook of the runtime): nothing faults, every rank leaves its kernel normally."""
    with _group(timeout_ms=300) as group:
        cpu, args = _inputs()
        ok = group.dispatch(*args, do_expand=True)
        assert all(code[0] == 0 for code in _codes(ok))
        del ok
        group.runtimes[1].set_test_corrupt_sequence(True)
        failed = group.dispatch(*args, do_expand=True)
        codes = _codes(failed)
        # whoever received a row of rank 1 refuses it (18, context = source rank 1); the others learn of the abort
        assert any(code[0] == 18 and code[1] == 1 for code in codes), codes
        assert all(code[0] in (0, 15, 18, 22) for code in codes), codes
        assert codes[1][0] in (0, 15, 22), codes  # the sender itself never reads its own rows from a ring
        del failed
        group.runtimes[1].set_test_corrupt_sequence(False)
        again = group.dispatch(*args, do_expand=True)
        assert any(code[0] == 19 for code in _codes(again))  # the failure is terminal for the ranks that saw it


def test_abort_published_in_mid_transfer_reaches_waiting_ranks(ext):
    """Rank 2 withholds its counts, so everybody waits; rank 1 publishes an abort 2 ms into the launch.  The
    waiting ranks leave with "peer abort" from rank 1 long before their own 5 s timeout would have fired."""
    import time

    with _group(timeout_ms=5000) as group:
        cpu, args = _inputs()
        ok = group.dispatch(*args, do_expand=True)
        assert all(code[0] == 0 for code in _codes(ok))
        del ok
        group.runtimes[2].set_test_withhold_counts(True)
        group.runtimes[1].set_test_control_abort_after_ns(2_000_000)
        started = time.perf_counter()
        failed = group.dispatch(*args, do_expand=True)
        codes = _codes(failed)
        elapsed = time.perf_counter() - started
        assert elapsed < 2.5, f"ranks waited {elapsed:.2f} s: the abort did not cut their waits short"
        assert any(code[0] == 22 and code[1] == 1 for code in codes), codes
        assert all(code[0] in (12, 22, 27) for code in codes), codes
