"""The conservative READY-flag publication on device segments (several ranks emulated on one GPU)."""

import pytest

from pcie_ep_b200 import HostStagedConfig
from tests.test_gpu_dispatch import _run_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("wire", ["bf16", "fp8_e4m3"])
def test_dispatch_with_one_fence_per_row_on_device_segments(ext, monkeypatch, wire):
    """The conservative publication (``PCIE_EP_B200_FENCE_EVERY_ROW=1``, read when the runtime is built): every send
    warp publishes row by row, each storing lane behind a fence of its own.  Same results as the batched default."""
    from pcie_ep_b200.parallel.virtual import VirtualEPGroup

    monkeypatch.setenv("PCIE_EP_B200_FENCE_EVERY_ROW", "1")
    world, experts, topk, hidden, tmax = 2, 16, 4, 1024, 64
    config = HostStagedConfig(channels=8, timeout_ms=5000, tx_warps=2, rx_warps=4, send_ctas=2, output_pool_size=2,
                              wire_dtype=wire, stage=7 if wire != "bf16" else 6)
    with VirtualEPGroup(world, tmax, hidden, topk, experts, config) as group:
        for repeat in range(3):
            results, _ = _run_case(group, world, experts, topk, hidden, tmax, [64, 49], "random", bool(repeat % 2), 1, seed=11 + repeat,
                                   wire=wire)
            del results
