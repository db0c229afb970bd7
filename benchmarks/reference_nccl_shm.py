"""Run the reference's own NCCL comparison (``benchmarks/benchmark_nccl_shm.py`` of yangshucan/PCIe-EP) on this box.

    python benchmarks/reference_nccl_shm.py --tokens 128 1024 4096 --output results/reference_nccl_shm

The reference script is used unmodified from ``baseline/_ref`` (a copy of the reference tree).  It compares three
variants on identical tensors at eight ranks: the reference's host-staged dispatch, a BF16 payload all-gather, and an
expert-ready dispatch (pack kernel, one uint8 all-gather, three expansion kernels).  At import it forces NCCL onto
shared memory (``NCCL_P2P_DISABLE=1``, ``NCCL_NVLS_ENABLE=0``, ...), because its target machines have no NVLink: its
numbers on an NVLink box are therefore "NCCL over host shared memory", and are recorded as such.  The NVLink-enabled
counterpart of the same three-way comparison is ``benchmarks/benchmark_nccl.py``.

This launcher only sets what the reference needs to run in this image: the sm_100 architecture for its JIT build,
an extension directory inside the repository (so that a build made ahead of time travels with it), and the system
libstdc++ preloaded (an extension built through ``torch.utils.cpp_extension`` here does not record libstdc++ as a
dependency, and the reference's ``std::ifstream`` use then binds to the wrong copy).
"""

from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
REFERENCE = ROOT / "baseline" / "_ref"


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--tokens", type=int, nargs="+", default=[128, 1024, 4096])
    parser.add_argument("--variants", nargs="+", default=["pcie_ep", "nccl_payload", "nccl_dispatch"])
    parser.add_argument("--iterations", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--output", type=Path, default=ROOT / "results" / "reference_nccl_shm")
    parser.add_argument("--port", type=int, default=29577)
    args = parser.parse_args()
    script = REFERENCE / "benchmarks" / "benchmark_nccl_shm.py"
    if not script.exists():
        print(f"{script} is missing: copy the reference tree to baseline/_ref first", file=sys.stderr)
        return 2
    env = dict(os.environ)
    env["TORCH_CUDA_ARCH_LIST"] = "10.0"
    env.setdefault("TORCH_EXTENSIONS_DIR", str(ROOT / "baseline" / "_ref_build"))
    env["PYTHONPATH"] = os.pathsep.join([str(REFERENCE), str(REFERENCE / "benchmarks"), env.get("PYTHONPATH", "")])
    preload = sorted(glob.glob("/usr/lib/x86_64-linux-gnu/libstdc++.so.6") + glob.glob("/usr/lib64/libstdc++.so.6"))
    if preload:
        env["LD_PRELOAD"] = preload[0] + (":" + env["LD_PRELOAD"] if env.get("LD_PRELOAD") else "")
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "8", "--master-addr", "127.0.0.1",
               "--master-port", str(args.port), str(script), "--tokens", *map(str, args.tokens), "--variants", *args.variants,
               "--iterations", str(args.iterations), "--warmup", str(args.warmup), "--topk", str(args.topk),
               "--output", str(args.output.resolve())]
    return subprocess.run(command, env=env, cwd=str(REFERENCE / "benchmarks")).returncode


if __name__ == "__main__":
    raise SystemExit(main())
