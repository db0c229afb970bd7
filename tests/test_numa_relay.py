"""The CPU relay against a scripted "GPU": the test writes what a sending kernel would write into an
outbox (counts message, staged rows, READY flags, hand-back flags, combine rows) and checks that the
relay threads reproduce it in the destination segment in protocol order.  Host memory only; the GPU
side of the same hand-off is covered by the host-staged relay run in test_gpu_multiprocess.py.
(reference: tests/test_relay.py checks copies == expected pairs and the drained epoch.)"""

import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")


def _wait(predicate, seconds=5.0):
    deadline = time.time() + seconds
    while time.time() < deadline:
        if predicate():
            return True
        time.sleep(0.002)
    return False


def test_relay_forwards_counts_rows_flags_and_combine(ext):
    P, C, E, K, H, TMAX = 2, 2, 8, 2, 64, 8
    lay = ext.segment_layout(P, C, E, K, H, TMAX, 0, True)
    size = int(lay["size_bytes"])
    outbox = np.zeros(size, dtype=np.uint8)
    target = np.zeros(size, dtype=np.uint8)
    unused = np.zeros(8, dtype=np.uint8)
    me, dest = 0, 1
    options = {"num_ranks": P, "channels": C, "num_experts": E, "num_topk": K, "hidden": H, "num_max_tokens": TMAX,
               "payload_slots": 0, "enable_combine": True, "workers": 1, "cpu_affinity": []}
    relay = ext.NumaRelay(options, [unused.ctypes.data, outbox.ctypes.data], [unused.ctypes.data, target.ctypes.data], me)
    relay.start()
    try:
        u64_out, u64_tgt = outbox.view(np.uint64), target.view(np.uint64)
        i32_out, i32_tgt = outbox.view(np.int32), target.view(np.int32)
        epoch = 1
        stride, row_stride, slots = int(lay["counts_stride"]), int(lay["row_stride"]), int(lay["slots"])
        # rows first (a fast channel may run ahead of the counts message): nothing may be forwarded yet
        chan_rows = [3, 1]
        rng = np.random.default_rng(0)
        for c, n in enumerate(chan_rows):
            for j in range(n):
                ring = (me * C + c) * slots + j
                at = int(lay["stage_off"]) + ring * row_stride
                outbox[at:at + int(lay["meta_off"]) + int(lay["meta_bytes"])] = rng.integers(0, 255, int(lay["meta_off"]) + int(lay["meta_bytes"]), dtype=np.uint8)
                u64_out[(int(lay["ready_off"]) + ring * 8) // 8] = (epoch << 32) | (j + 1)
        time.sleep(0.05)
        assert relay.diagnostics()["flows"][0]["rows_copied"] == 0
        # counts message: rank counts | expert counts | channel counts, then its flag
        base = (int(lay["counts_off"]) + me * stride * 4) // 4
        message = np.arange(stride, dtype=np.int32)
        message[P + E // P:P + E // P + C] = chan_rows
        i32_out[base:base + stride] = message
        u64_out[(int(lay["counts_flag_off"]) + me * 32) // 8] = epoch
        assert _wait(lambda: relay.diagnostics()["flows"][0]["rows_copied"] == sum(chan_rows))
        assert u64_tgt[(int(lay["counts_flag_off"]) + me * 32) // 8] == epoch
        assert np.array_equal(i32_tgt[base:base + stride], message)
        for c, n in enumerate(chan_rows):
            for j in range(n):
                ring = (me * C + c) * slots + j
                at = int(lay["stage_off"]) + ring * row_stride
                width = int(lay["meta_off"]) + int(lay["meta_bytes"])
                assert np.array_equal(target[at:at + width], outbox[at:at + width])
                assert u64_tgt[(int(lay["ready_off"]) + ring * 8) // 8] == (epoch << 32) | (j + 1)
        # hand-backs and abort
        u64_out[(int(lay["done_off"]) + me * 32) // 8] = 1
        u64_out[(int(lay["cdone_off"]) + me * 32) // 8] = 1
        assert _wait(lambda: u64_tgt[(int(lay["done_off"]) + me * 32) // 8] == 1 and u64_tgt[(int(lay["cdone_off"]) + me * 32) // 8] == 1)
        # a combine row for token 5
        crow = int(lay["crow_stride"])
        at = int(lay["cstage_off"]) + (me * TMAX + 5) * crow
        outbox[at:at + H * 2] = rng.integers(0, 255, H * 2, dtype=np.uint8)
        u64_out[(int(lay["cready_off"]) + (me * TMAX + 5) * 8) // 8] = 1
        assert _wait(lambda: u64_tgt[(int(lay["cready_off"]) + (me * TMAX + 5) * 8) // 8] == 1)
        assert np.array_equal(target[at:at + H * 2], outbox[at:at + H * 2])
        u64_out[(int(lay["abort_off"]) + me * 32) // 8] = 15
        assert _wait(lambda: u64_tgt[(int(lay["abort_off"]) + me * 32) // 8] == 15)
        flow = relay.diagnostics()["flows"][0]
        assert flow["dest"] == dest and flow["failure"] == 0 and flow["combine_rows_copied"] == 1 and flow["counts_epoch"] == 1
    finally:
        relay.stop()
    assert not relay.diagnostics()["running"]


def test_relay_flags_overfull_counts(ext):
    options = {"num_ranks": 2, "channels": 1, "num_experts": 4, "num_topk": 2, "hidden": 32, "num_max_tokens": 8,
               "payload_slots": 0, "enable_combine": False, "workers": 1, "cpu_affinity": []}
    buf = np.zeros(8, dtype=np.uint8)
    lay = ext.segment_layout(2, 1, 4, 2, 32, 8, 0, False)
    outbox = np.zeros(int(lay["size_bytes"]), dtype=np.uint8)
    target = np.zeros(int(lay["size_bytes"]), dtype=np.uint8)
    relay = ext.NumaRelay(options, [buf.ctypes.data, outbox.ctypes.data], [buf.ctypes.data, target.ctypes.data], 0)
    relay.start()
    try:
        i32 = outbox.view(np.int32)
        base = int(lay["counts_off"]) // 4
        i32[base + 2 + 2] = 99  # more rows than a channel can ever hold
        outbox.view(np.uint64)[int(lay["counts_flag_off"]) // 8] = 1
        assert _wait(lambda: relay.diagnostics()["flows"][0]["failure"] == 102)
    finally:
        relay.stop()


def test_relay_bounded_ring_waits_for_credit_and_forwards_acks(ext):
    """Two-slot rings: the relay copies rows 0 and 1, holds row 2 back until the destination's acknowledgement of
    row 0 has reached this rank's own segment, and forwards the acknowledgements this rank's GPU writes for rows
    it received to the peer."""
    P, C, E, K, H, TMAX, Q = 2, 1, 4, 2, 32, 8, 2
    lay = ext.segment_layout(P, C, E, K, H, TMAX, Q, False)
    assert int(lay["slots"]) == Q and int(lay["slots_full"]) == TMAX
    size = int(lay["size_bytes"])
    own = np.zeros(size, dtype=np.uint8)      # this rank's real segment: credit arrives here
    outbox = np.zeros(size, dtype=np.uint8)   # what this rank's GPU writes towards rank 1
    target = np.zeros(size, dtype=np.uint8)   # rank 1's real segment
    me, dest, epoch = 0, 1, 1
    options = {"num_ranks": P, "channels": C, "num_experts": E, "num_topk": K, "hidden": H, "num_max_tokens": TMAX,
               "payload_slots": Q, "enable_combine": False, "workers": 1, "cpu_affinity": [], "target_numa_nodes": [0, 0]}
    relay = ext.NumaRelay(options, [own.ctypes.data, outbox.ctypes.data], [own.ctypes.data, target.ctypes.data], me)
    relay.start()
    try:
        assert relay.diagnostics()["ring_mode"]
        u64_out, u64_tgt, u64_own = outbox.view(np.uint64), target.view(np.uint64), own.view(np.uint64)
        stride, row_stride = int(lay["counts_stride"]), int(lay["row_stride"])
        width = int(lay["meta_off"]) + int(lay["meta_bytes"])
        message = np.zeros(stride, dtype=np.int32)
        message[P + E // P] = 3  # channel 0 will carry three rows
        base = (int(lay["counts_off"]) + me * stride * 4) // 4
        outbox.view(np.int32)[base:base + stride] = message
        u64_out[(int(lay["counts_flag_off"]) + me * 32) // 8] = epoch

        def publish(j, fill):
            ring = (me * C + 0) * Q + j % Q
            at = int(lay["stage_off"]) + ring * row_stride
            outbox[at:at + width] = fill
            u64_out[(int(lay["ready_off"]) + ring * 8) // 8] = (epoch << 32) | (j + 1)

        publish(0, 11)
        publish(1, 22)
        assert _wait(lambda: relay.diagnostics()["flows"][0]["rows_copied"] == 2)
        publish(2, 33)  # reuses slot 0: must wait for the acknowledgement of row 0
        time.sleep(0.05)
        flow = relay.diagnostics()["flows"][0]
        assert flow["rows_copied"] == 2 and flow["credit_waits"] > 0 and flow["drained_epoch"] == 0
        slot0 = int(lay["stage_off"]) + (me * C) * Q * row_stride
        assert target[slot0] == 11  # row 0 is still intact at the destination
        # the destination acknowledges row 0: the flag lands in this rank's own segment, indexed by the destination
        u64_own[(int(lay["ack_off"]) + ((dest * C + 0) * Q + 0) * 8) // 8] = (epoch << 32) | 1
        assert _wait(lambda: relay.diagnostics()["flows"][0]["rows_copied"] == 3)
        assert target[slot0] == 33 and relay.diagnostics()["flows"][0]["drained_epoch"] == epoch
        # an acknowledgement written by this rank's GPU (as a destination of rank 1) travels the other way
        ack_index = (int(lay["ack_off"]) + ((me * C + 0) * Q + 1) * 8) // 8
        u64_out[ack_index] = (epoch << 32) | 2
        assert _wait(lambda: u64_tgt[ack_index] == ((epoch << 32) | 2))
        assert relay.diagnostics()["flows"][0]["acks_forwarded"] == 1
    finally:
        relay.stop()


def test_relay_groups_workers_by_numa_node(ext):
    P = 4
    lay = ext.segment_layout(P, 1, 4, 2, 32, 8, 0, False)
    size = int(lay["size_bytes"])
    boxes = [np.zeros(size, dtype=np.uint8) for _ in range(2 * P)]
    options = {"num_ranks": P, "channels": 1, "num_experts": 4, "num_topk": 2, "hidden": 32, "num_max_tokens": 8,
               "payload_slots": 0, "enable_combine": False, "workers": 1, "cpu_affinity": [], "target_numa_nodes": [0, 0, 1, 1]}
    relay = ext.NumaRelay(options, [b.ctypes.data for b in boxes[:P]], [b.ctypes.data for b in boxes[P:]], 0)
    relay.start()
    try:
        info = relay.diagnostics()
        assert info["workers"] == 2  # one worker per NUMA node that has destinations (ranks 1 | 2, 3)
        assert sorted((f["dest"], f["numa_node"]) for f in info["flows"]) == [(1, 0), (2, 1), (3, 1)]
    finally:
        relay.stop()


def test_query_numa_pages_counts_every_page(ext):
    import mmap

    pages = 16
    buf = np.zeros(pages * mmap.PAGESIZE, dtype=np.uint8)
    buf[:] = 1  # touched: every page is resident somewhere
    placement = ext.query_numa_pages(buf.ctypes.data, buf.nbytes)
    assert sum(placement.values()) in (pages, pages + 1)  # +1 when the array is not page-aligned
    assert all(isinstance(node, int) and node >= -1 for node in placement)


def test_explicit_relay_cpus_are_a_restriction_not_a_wish(ext):
    """``cpu_affinity``: workers run on the named CPUs that lie on the destination's NUMA node and that the process may
    use; if none is left, construction fails (on every rank alike, through the buffer's agreement round)."""
    import os

    P, C, E, K, H, TMAX = 2, 2, 8, 2, 64, 8
    lay = ext.segment_layout(P, C, E, K, H, TMAX, 0, False)
    size = int(lay["size_bytes"])
    outbox, target, unused = (np.zeros(size, dtype=np.uint8), np.zeros(size, dtype=np.uint8), np.zeros(8, dtype=np.uint8))
    options = {"num_ranks": P, "channels": C, "num_experts": E, "num_topk": K, "hidden": H, "num_max_tokens": TMAX,
               "payload_slots": 0, "enable_combine": False, "workers": 1}
    pointers = ([unused.ctypes.data, outbox.ctypes.data], [unused.ctypes.data, target.ctypes.data], 0)
    usable = sorted(os.sched_getaffinity(0))
    chosen = usable[-1]
    relay = ext.NumaRelay(dict(options, cpu_affinity=[chosen, 100000]), *pointers)     # an impossible CPU beside a usable one
    relay.start()
    try:
        assert _wait(lambda: relay.diagnostics()["flows"][0]["worker_cpu"] == chosen)
    finally:
        relay.stop()
    with pytest.raises(ValueError, match="no usable CPU"):
        ext.NumaRelay(dict(options, cpu_affinity=[100000]), *pointers)
