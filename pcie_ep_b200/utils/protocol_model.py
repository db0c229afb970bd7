"""Builds and runs the host model of the dispatch and combine protocol (``csrc/model/protocol_model.cpp``).

    python -m pcie_ep_b200.utils.protocol_model --ranks 4 --slots 2 --epochs 6 --delay-us 20
    python -m pcie_ep_b200.utils.protocol_model --sanitize --publish relaxed        # ThreadSanitizer names the race
    python -m pcie_ep_b200.utils.protocol_model --withhold-counts 1 --timeout-ms 300 --expect 12
    python -m pcie_ep_b200.utils.protocol_model --combine 1 --withhold-signal 2 --timeout-ms 800 --expect 25
    python -m pcie_ep_b200.utils.protocol_model --sanitize --relay 1 --slots 2      # the product's CPU relay in the middle

Ranks are threads, segments are host memory with the kernels' own layout, flags are ``std::atomic_ref``: the
protocol's rules run under ThreadSanitizer, and the failure scenarios that must not be staged on a shared GPU
(a rank that never sends counts, never returns credit, never hands its staging or landing area back, writes a wrong
sequence, never signals its combine rows)
run on the CPU.  The program prints one JSON object per rank.
"""

from __future__ import annotations

import json
import shutil
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

_ROOT = Path(__file__).resolve().parents[2]
_SOURCE = _ROOT / "csrc" / "model" / "protocol_model.cpp"
_OUT = Path(__file__).resolve().parents[1] / "_ext" / "model"


def _cuda_include() -> List[str]:
    for candidate in ("/usr/local/cuda/include",):
        if Path(candidate, "cuda_runtime.h").exists():
            return ["-I" + candidate]
    nvcc = shutil.which("nvcc")
    if nvcc:
        return ["-I" + str(Path(nvcc).resolve().parents[1] / "include")]
    return []


def build(sanitize=False) -> Path:
    """Compile the model with the host compiler; returns the executable.  ``sanitize``: False, True or ``"thread"``
    (ThreadSanitizer), ``"address"`` (AddressSanitizer + UndefinedBehaviorSanitizer)."""
    compiler = shutil.which("g++")
    if compiler is None:
        raise RuntimeError("no g++ on PATH")
    kind = "thread" if sanitize is True else (sanitize or "")
    if kind not in ("", "thread", "address"):
        raise ValueError("sanitize is False, True, 'thread' or 'address'")
    _OUT.mkdir(parents=True, exist_ok=True)
    target = _OUT / {"": "protocol_model", "thread": "protocol_model_tsan", "address": "protocol_model_asan"}[kind]
    headers = [_ROOT / "csrc" / "kernels" / "protocol.cuh", _ROOT / "csrc" / "comm" / "numa_relay.hpp", _SOURCE]
    if target.exists() and all(target.stat().st_mtime >= h.stat().st_mtime for h in headers):
        return target
    command = [compiler, "-std=c++20", "-O1", "-g", "-pthread", "-Wno-tsan", "-I" + str(_ROOT / "csrc"), *_cuda_include()]
    if kind == "thread":
        command.append("-fsanitize=thread")
    elif kind == "address":
        command += ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
    command += [str(_SOURCE), "-o", str(target)]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError("building the protocol model failed:\n" + done.stderr[-2000:])
    return target


def run_with_summary(arguments: Sequence[str], sanitize=False, timeout: float = 120.0) -> Tuple[int, List[Dict], Dict, str]:
    """(exit status, one dict per rank, the relay's summary line or {}, stderr).  Under the sanitizer a reported race
    makes the status non-zero."""
    done = subprocess.run([str(build(sanitize)), *map(str, arguments)], capture_output=True, text=True, timeout=timeout)
    records = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    ranks = [r for r in records if "rank" in r]
    summary = next((r for r in records if "relay_rows" in r), {})
    return done.returncode, ranks, summary, done.stderr


def run(arguments: Sequence[str], sanitize=False, timeout: float = 120.0) -> Tuple[int, List[Dict], str]:
    """(exit status, one dict per rank, stderr)."""
    status, ranks, _, stderr = run_with_summary(arguments, sanitize, timeout)
    return status, ranks, stderr


def main() -> None:
    arguments = sys.argv[1:]
    sanitize = "address" if "--sanitize-address" in arguments else "--sanitize" in arguments
    arguments = [a for a in arguments if a not in ("--sanitize", "--sanitize-address")]
    status, ranks, summary, stderr = run_with_summary(arguments, sanitize)
    for rank in ranks:
        print(json.dumps(rank))
    if summary:
        print(json.dumps(summary))
    if stderr:
        print(stderr[-3000:], file=sys.stderr)
    raise SystemExit(status)


if __name__ == "__main__":
    main()
