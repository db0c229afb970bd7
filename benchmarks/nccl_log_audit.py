"""Which transport did NCCL use?  Reads ``NCCL_DEBUG=INFO`` logs of a baseline run and says so.

    NCCL_DEBUG=INFO NCCL_DEBUG_FILE=results/nccl.%h.%p.log python -m torch.distributed.run ... benchmarks/benchmark_nccl.py ...
    python benchmarks/nccl_log_audit.py --expect nvlink --world 8 results/nccl.*.log

A comparison with NCCL is only worth something if NCCL ran over the path the comparison claims.  The NVLink-enabled
baseline of this repository (``benchmarks/benchmark_nccl.py``) must show peer-to-peer connections (and may show NVLS),
never shared memory or the network; the reference's own baseline (``benchmarks/reference_nccl_shm.py``) forces shared
memory, and then every connection must be SHM.  ``--expect`` names which of the two is being checked.

What is kept from the logs: the NCCL version, how many ranks finished initialisation, and per transport family the
number of connection lines and of distinct (source, destination) pairs.  No host name, process id, address or path of a
log enters the result.  Exit status 0: as expected; 1: not; 2: the logs do not contain what the audit needs.

Parity: the reference's ``scripts/check_nccl_shm_logs.py`` (all connections SHM, nothing else), here for both directions.
"""

from __future__ import annotations

import argparse
import json
import re
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, Iterable, List

FAMILIES = ("P2P", "SHM", "NET", "NVLS", "COLLNET")

_MESSAGE = re.compile(r"NCCL INFO\s+(.*)$")
_VERSION = re.compile(r"NCCL version\s+(\d+\.\d+\.\d+)")
_INIT_DONE = re.compile(r"rank\s+(\d+)\s+nranks\s+(\d+)\b.*Init COMPLETE")
_CONNECTION = re.compile(r"^Channel\s+\d+(?:/\d+)?\s*:\s*(\d+)\[[^\]]*\]\s*->\s*(\d+)\[[^\]]*\].*?\bvia\s+([A-Za-z0-9]+)")
_NVLS_ACTIVE = re.compile(r"NVLS (?:Creat\w+ Multicast group|importing shareableHandle|comm\b)|Connected NVLS tree")


def summarise(texts: Iterable[str]) -> Dict:
    """Counts from the text of one or more log files (one per process, or one for all)."""
    versions, ranks_done, sizes = set(), set(), set()
    lines_by_family: Dict[str, int] = defaultdict(int)
    pairs_by_family: Dict[str, set] = defaultdict(set)
    nvls_active = False
    for text in texts:
        for raw in text.splitlines():
            version = _VERSION.search(raw)   # (printed with and without the INFO prefix, depending on the NCCL version)
            if version:
                versions.add(version.group(1))
            found = _MESSAGE.search(raw)
            if not found:
                continue
            message = found.group(1).strip()
            done = _INIT_DONE.search(message)
            if done:
                ranks_done.add(int(done.group(1)))
                sizes.add(int(done.group(2)))
            if _NVLS_ACTIVE.search(message):
                nvls_active = True
            connection = _CONNECTION.match(message)
            if connection:
                family = connection.group(3).upper()
                family = family if family in FAMILIES else "OTHER"
                lines_by_family[family] += 1
                pairs_by_family[family].add((int(connection.group(1)), int(connection.group(2))))
    return {
        "nccl_versions": sorted(versions),
        "ranks_initialised": len(ranks_done),
        "communicator_sizes": sorted(sizes),
        "connection_lines": dict(sorted(lines_by_family.items())),
        "connected_pairs": {family: len(pairs) for family, pairs in sorted(pairs_by_family.items())},
        "nvls_active": nvls_active,
    }


def verdict(summary: Dict, expect: str, world: int) -> List[str]:
    """Reasons why the logs do not show what ``expect`` ("nvlink" or "shm") claims; empty when they do."""
    problems = []
    lines = summary["connection_lines"]
    if summary["ranks_initialised"] < world:
        problems.append(f"{summary['ranks_initialised']} of {world} ranks report a finished initialisation")
    if not lines and not summary["nvls_active"]:
        problems.append("no connection lines: was NCCL_DEBUG=INFO (with INIT or ALL subsystems) set?")
        return problems
    if expect == "nvlink":
        if lines.get("P2P", 0) == 0 and not summary["nvls_active"]:
            problems.append("no peer-to-peer connection and no NVLS: NCCL did not use NVLink")
        for family in ("SHM", "NET", "OTHER"):
            if lines.get(family, 0):
                problems.append(f"{lines[family]} connection line(s) via {family}")
    elif expect == "shm":
        if lines.get("SHM", 0) == 0:
            problems.append("no shared-memory connection")
        for family in ("P2P", "NET", "NVLS", "COLLNET", "OTHER"):
            if lines.get(family, 0):
                problems.append(f"{lines[family]} connection line(s) via {family}")
        if summary["nvls_active"]:
            problems.append("NVLS was set up")
    else:
        raise ValueError("expect is 'nvlink' or 'shm'")
    return problems


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("logs", nargs="+", type=Path)
    parser.add_argument("--expect", required=True, choices=["nvlink", "shm"])
    parser.add_argument("--world", type=int, required=True, help="ranks of the run the logs belong to")
    args = parser.parse_args(argv)
    summary = summarise(path.read_text(errors="replace") for path in args.logs)
    problems = verdict(summary, args.expect, args.world)
    print(json.dumps({"expect": args.expect, "world": args.world, "logs": len(args.logs), **summary, "problems": problems}, indent=2))
    if problems and (not summary["connection_lines"] and not summary["nvls_active"]):
        return 2
    return 1 if problems else 0


if __name__ == "__main__":
    raise SystemExit(main())
