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


def test_relay_rejects_bounded_rings_and_flags_overfull_counts(ext):
    options = {"num_ranks": 2, "channels": 1, "num_experts": 4, "num_topk": 2, "hidden": 32, "num_max_tokens": 8,
               "payload_slots": 2, "enable_combine": False, "workers": 1, "cpu_affinity": []}
    buf = np.zeros(8, dtype=np.uint8)
    with pytest.raises(ValueError):
        ext.NumaRelay(options, [buf.ctypes.data] * 2, [buf.ctypes.data] * 2, 0)
    options["payload_slots"] = 0
    lay = ext.segment_layout(2, 1, 4, 2, 32, 8, 0, False)
    outbox = np.zeros(int(lay["size_bytes"]), dtype=np.uint8)
    target = np.zeros(int(lay["size_bytes"]), dtype=np.uint8)
    relay = ext.NumaRelay(options, [buf.ctypes.data, outbox.ctypes.data], [buf.ctypes.data, target.ctypes.data], 0)
    relay.start()
    try:
        i32 = outbox.view(np.int32)
        base = int(lay["counts_off"]) // 4
        i32[base + 2 + 2] = 99  # more rows than the ring holds
        outbox.view(np.uint64)[int(lay["counts_flag_off"]) // 8] = 1
        assert _wait(lambda: relay.diagnostics()["flows"][0]["failure"] == 102)
    finally:
        relay.stop()
