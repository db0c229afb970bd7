"""CPU (gloo) transport through the public API, world size 2 and 4, as real processes."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

from tests.helpers import free_port

ROOT = Path(__file__).resolve().parents[1]


def run_workers(world, *extra, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           str(ROOT / "tests" / "workers" / "ep_worker.py"), *extra]
    proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "OK suite=" in proc.stdout
    return proc.stdout


@pytest.mark.parametrize("world", [2, 4, 8])
def test_cpu_transport_correctness(world):
    run_workers(world, "--transport", "cpu", "--suite", "correctness", "--hidden", "64", "--small")


def test_cpu_transport_oracle_config_world2():
    """world_size=2, T=64, hidden=128, fp32, 8 experts, top-2."""
    run_workers(2, "--transport", "cpu", "--suite", "oracle_config", "--fp32")


def test_cpu_moe_layer_world2():
    run_workers(2, "--transport", "cpu", "--suite", "moe_layer", "--hidden", "64")


def test_cpu_moe_layer_with_fused_expert_combine_api_world2():
    """The fused call exists on every transport; on CPU it is the two-step evaluation."""
    run_workers(2, "--transport", "cpu", "--suite", "moe_layer", "--hidden", "64", "--fused-layer")


def test_the_example_runs_on_two_cpu_ranks():
    """examples/moe_exchange.py: route, dispatch, local experts, combine, checked against the closed form."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), str(ROOT / "examples" / "moe_exchange.py"), "--tokens", "48", "--hidden", "128"]
    proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "largest deviation from the closed form" in proc.stdout
