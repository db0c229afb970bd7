"""Recompute comparison tables from saved benchmark records (CPU only).

    python benchmarks/report.py results/eager.json results/graph.json --baseline published

Inputs are the JSON files written by ``benchmarks/benchmark.py --output``.  Records are only compared
when their shape arguments agree (hidden, experts, top-k, world, profile, wire); anything else is
refused rather than silently mixed -- the rule of the reference's report tools
(``benchmarks/report_latest.py``, ``report_control_progress.py`` there).  ``--baseline published`` adds
the reference's published dispatch latencies (8x H20D, PCIe 5; ``RESULTS_CONTROL_PROGRESS.md:31-40``).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Dict, List

PUBLISHED_US = {16: 260, 32: 282, 64: 405, 128: 647, 256: 1033, 512: 1950, 1024: 3681, 2048: 7079, 4096: 13558, 8192: 26546}
SHAPE_KEYS = ("hidden", "experts", "topk", "profile", "wire")


def load(path: Path) -> Dict:
    data = json.loads(Path(path).read_text())
    if "records" not in data or "arguments" not in data:
        raise ValueError(f"{path}: not a benchmark record file")
    return data


def check_comparable(files: List[Dict]) -> None:
    first = files[0]
    for other in files[1:]:
        for key in SHAPE_KEYS:
            if str(first["arguments"].get(key)) != str(other["arguments"].get(key)):
                raise ValueError(f"records disagree on {key!r}: {first['arguments'].get(key)} vs {other['arguments'].get(key)}")
        worlds = {r["world"] for r in first["records"]} | {r["world"] for r in other["records"]}
        if len(worlds) != 1:
            raise ValueError(f"records come from different world sizes: {sorted(worlds)}")


def table(files: List[Dict], labels: List[str], baseline: str = "") -> str:
    check_comparable(files)
    tokens = sorted({r["tokens"] for f in files for r in f["records"]})
    header = ["T"] + [f"{label} dispatch us" for label in labels] + [f"{label} combine us" for label in labels]
    if baseline == "published":
        header += ["published reference us", "speedup (first column)"]
    lines = ["| " + " | ".join(header) + " |", "|" + "---|" * len(header)]
    for t in tokens:
        row = [str(t)]
        dispatch = []
        for f in files:
            rec = next((r for r in f["records"] if r["tokens"] == t), None)
            dispatch.append(rec["dispatch_us_mean"] if rec else None)
            row.append(f"{rec['dispatch_us_mean']:.1f}" if rec else "-")
        for f in files:
            rec = next((r for r in f["records"] if r["tokens"] == t), None)
            row.append(f"{rec['combine_us_mean']:.1f}" if rec and rec.get("combine_us_mean") is not None else "-")
        if baseline == "published":
            ref = PUBLISHED_US.get(t)
            row.append(str(ref) if ref else "-")
            row.append(f"{ref / dispatch[0]:.1f}x" if ref and dispatch[0] else "-")
        lines.append("| " + " | ".join(row) + " |")
    return "\n".join(lines)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("files", type=Path, nargs="+")
    parser.add_argument("--baseline", default="", choices=["", "published"])
    args = parser.parse_args()
    files = [load(p) for p in args.files]
    print(table(files, [p.stem for p in args.files], args.baseline))


if __name__ == "__main__":
    main()
