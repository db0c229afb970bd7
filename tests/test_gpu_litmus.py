"""READY/ACK publication litmus (parity: the reference's tests/mapped_litmus.cu + MAPPED_LITMUS.md): payload stores,
st.release.sys of a single-writer flag, ld.acquire.sys + payload check on the other side, ACK back; and the same
round trip with the payload pushed by cp.async.bulk and the flag stored after the bulk group's completion.
One GPU: both sides as two CTAs of one cooperative launch.  Two GPUs: one process per side over IPC."""

import pytest
import torch

from tests.test_cpu_transport import run_workers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("method", [0, 1])
def test_litmus_two_ctas_one_gpu(ext, method):
    """method 0: ordinary stores + st.release.sys; method 1: bulk copy, completion wait, system fence, relaxed flag (the send warps' chain)."""
    size, rounds, words = 1 << 16, 50000 if method == 0 else 20000, 512
    a = ext.allocate_device_segment(size, 0)
    b = ext.allocate_device_segment(size, 0)
    status = torch.zeros(8, dtype=torch.int64, device="cuda")
    ext.litmus(a, b, -1, rounds, words, status, 5000, 0, method)
    torch.cuda.synchronize()
    producer, consumer = status[:4].tolist(), status[4:].tolist()
    assert producer[0] == 0 and consumer[0] == 0, "a bounded wait expired"
    assert consumer[1] == 0, f"{consumer[1]} payload words were stale when READY was visible"
    assert producer[2] == rounds and consumer[2] == rounds
    ext.free_device_segment(a)
    ext.free_device_segment(b)


def test_litmus_wait_gives_up_without_a_partner(ext):
    """A flag that nothing sets: the wait runs out after its limit and the kernel reports it."""
    a = ext.allocate_device_segment(1 << 16, 0)
    b = ext.allocate_device_segment(1 << 16, 0)
    status = torch.zeros(4, dtype=torch.int64, device="cuda")
    ext.litmus(a, b, 1, 10, 64, status, 50, 0)  # a consumer alone, 50 ms limit
    torch.cuda.synchronize()
    assert status.tolist()[0] == 1 and status.tolist()[2] == 0
    torch.zeros(1, device="cuda").add_(1)  # the context is still usable
    torch.cuda.synchronize()
    ext.free_device_segment(a)
    ext.free_device_segment(b)


def test_litmus_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = run_workers(2, "--transport", "peer", "--suite", "litmus")
    assert "litmus:" in out
