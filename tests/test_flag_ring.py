"""The send warps' ring of READY flags that wait for their fence: a step-by-step model of its index arithmetic.

The dispatch kernel keeps the flags of rows whose bulk copies may still be in flight in a register ring of
``kFlagBatch + kFlagLag`` entries, publishes all but the ``kFlagLag`` newest whenever ``flag_batch`` rows have been issued
since the last publication (after waiting for all but the ``kFlagLag`` newest copy groups), publishes everything before a
credit wait and at the end.  The model below follows those rules with the constants read from the kernel's header and
checks, for every batch size and row count, that each flag goes out exactly once, in row order, never before its copy
group is known to be complete, and that no entry is pushed out of the ring unpublished."""

import random
import re
from pathlib import Path

import pytest

KERNELS = Path(__file__).resolve().parents[1] / "csrc" / "kernels"
HEADER = (KERNELS / "dispatch_common.cuh").read_text() + (KERNELS / "dispatch_send.cuh").read_text()


def constant(name: str) -> int:
    return int(re.search(rf"constexpr int {name} = (\d+);", HEADER).group(1))


LAG, BATCH = constant("kFlagLag"), constant("kFlagBatch")


def simulate(rows: int, flag_batch: int, credit_waits=()):
    ring = [None] * (BATCH + LAG)
    published, complete_upto, since = [], -1, 0   # complete_upto: newest row whose copy group is known to be complete

    def publish(entries, upto):
        nonlocal complete_upto
        complete_upto = max(complete_upto, upto)
        for i in entries:
            if ring[i] is not None:
                assert ring[i] <= complete_upto, "a flag left before its row's copies were complete"
                published.append(ring[i])
                ring[i] = None

    for n in range(rows):
        if n in credit_waits:                       # wait for every group, fence, publish everything held back
            publish(range(len(ring)), n - 1)
            since = 0
        assert ring[0] is None, "an unpublished flag was pushed out of the ring"
        ring[:] = ring[1:] + [n]
        since += 1
        if since >= flag_batch and n >= LAG:        # wait for all but the LAG newest groups, fence, publish the rest
            publish(range(len(ring) - LAG), n - LAG)
            since = 0
    publish(range(len(ring)), rows - 1)             # drain
    return published


def test_the_header_sizes_the_ring_for_its_batch_and_lag():
    assert re.search(r"constexpr int kRing = kFlagBatch \+ kFlagLag;", HEADER)
    assert re.search(r"flag_batch = fence_flags \? 1 : max\(1, min\(kFlagBatch,", HEADER)   # never more rows per fence than the ring allows


@pytest.mark.parametrize("flag_batch", range(1, BATCH + 1))
def test_every_flag_goes_out_once_in_order_and_only_after_its_copies(flag_batch):
    for rows in range(0, 4 * (BATCH + LAG) + 3):
        assert simulate(rows, flag_batch) == list(range(rows))
    rng = random.Random(flag_batch)
    for _ in range(200):
        rows = rng.randrange(1, 80)
        waits = {n for n in range(rows) if rng.random() < 0.15}
        assert simulate(rows, flag_batch, waits) == list(range(rows))


def test_a_batch_larger_than_the_ring_allows_would_lose_flags():
    """The check has teeth: one more row per fence than the ring holds pushes an unpublished flag out."""
    with pytest.raises(AssertionError, match="pushed out"):
        simulate(40, BATCH + 1)
