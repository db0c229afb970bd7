"""One process per GPU through the public API: peer-memory transport over NVLink (CUDA IPC) and the
host-staged fallback.  World size 1 always runs; larger worlds run when the box has the GPUs."""

import pytest
import torch

from tests.test_cpu_transport import run_workers

pytestmark = pytest.mark.gpu


def _need(gpus):
    if torch.cuda.device_count() < gpus:
        pytest.skip(f"needs {gpus} GPUs")


@pytest.mark.parametrize("transport", ["peer", "host_staged"])
def test_single_rank_public_api(transport):
    run_workers(1, "--transport", transport, "--suite", "correctness", "--hidden", "256")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_transport_correctness(world):
    _need(world)
    run_workers(world, "--transport", "peer", "--suite", "correctness", "--hidden", "512")


def test_peer_transport_bounded_ring_world2():
    _need(2)
    run_workers(2, "--transport", "peer", "--suite", "correctness", "--hidden", "256", "--payload-slots", "2")


def test_host_staged_transport_world2():
    _need(2)
    run_workers(2, "--transport", "host_staged", "--suite", "correctness", "--hidden", "256")


def test_oracle_config_on_gpus():
    _need(2)
    run_workers(2, "--transport", "peer", "--suite", "oracle_config")


def test_moe_layer_single_gpu():
    run_workers(1, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256")


@pytest.mark.parametrize("world", [2, 8])
def test_moe_layer_multi_gpu(world):
    _need(world)
    run_workers(world, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256")


def test_host_staged_relay_world2():
    """GPU -> own outbox -> CPU relay threads -> destination segment -> destination GPU."""
    _need(2)
    run_workers(2, "--transport", "host_staged", "--numa-mode", "relay", "--suite", "correctness", "--hidden", "256")


def test_moe_layer_fp8_path_single_gpu():
    """FP8 wire kept at the receiver + kind::f8f6f4 gate/up GEMM, against the same quantisation done in PyTorch."""
    run_workers(1, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256", "--fp8-layer")


def test_moe_layer_fp8_path_two_gpus():
    _need(2)
    run_workers(2, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256", "--fp8-layer")


def test_moe_layer_fused_down_projection_and_combine_single_gpu():
    """The GEMM epilogue writes into the (here: own) landing area; the owner-side reduction finishes the layer."""
    run_workers(1, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256", "--fused-layer")


@pytest.mark.parametrize("world", [2, 8])
def test_moe_layer_fused_down_projection_and_combine_multi_gpu(world):
    """Same over NVLink: tensor-core tiles and peer stores in one kernel, signalled to the owners by its last CTA."""
    _need(world)
    run_workers(world, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256", "--fused-layer")


def test_moe_layer_fused_with_fp8_dispatch_two_gpus():
    _need(2)
    run_workers(2, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256", "--fp8-layer", "--fused-layer")


@pytest.mark.parametrize("world,mode", [(2, "inline"), (2, "separate"), (4, "inline"), (8, "inline")])
def test_combine_owner_side_modes_across_processes(world, mode):
    """Both owner-side modes of combine (auto picks separate with more than one rank, so the other suites cover
    that one at every size): full correctness suite, one process per GPU, flags crossing NVLink."""
    _need(world)
    run_workers(world, "--transport", "peer", "--suite", "correctness", "--hidden", "256", "--combine-reduce", mode)


def test_moe_layer_with_separate_combine_reduction_two_gpus():
    _need(2)
    run_workers(2, "--transport", "peer", "--suite", "moe_layer", "--hidden", "256", "--combine-reduce", "separate")


def test_large_payload_headline_shape():
    """T=4096 tokens per rank at hidden 7168 / 256 experts / top-8 on every GPU of the box (2, 4 or 8): every received
    row is compared with its regenerated source, BF16 and FP8 wire, plus dedup counters and the combine round trip."""
    gpus = torch.cuda.device_count()
    world = 8 if gpus >= 8 else 4 if gpus >= 4 else 2 if gpus >= 2 else 0
    if world == 0:
        pytest.skip("needs at least 2 GPUs")
    out = run_workers(world, "--transport", "peer", "--suite", "large", "--tokens", "4096", "--timeout-ms", "20000")
    assert "large:" in out
