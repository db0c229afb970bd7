"""Recompute comparison tables from saved benchmark records (CPU only).

    python benchmarks/report.py results/eager.json results/graph.json --baseline published
    python benchmarks/report.py --bench benchmarks/data/results/bench_*gpu*.json      # scaling + sweep tables from bench.py lines

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


def load_bench_line(path: Path) -> Dict:
    """The JSON line that ``bench.py`` prints (the last line of a saved log that parses as JSON with a ``metric``)."""
    for line in reversed(Path(path).read_text().splitlines()):
        line = line.strip()
        if line.startswith("{"):
            try:
                record = json.loads(line)
            except json.JSONDecodeError:
                continue
            if "metric" in record or "unavailable" in record:
                return record
    raise ValueError(f"{path}: no bench.py result line")


def scaling_table(records: List[Dict]) -> str:
    """Weak-scaling table from ``bench.py`` lines of one implementation at several GPU counts.

    Lines are only put side by side when metric, unit, dtype and the model part of ``config`` agree.  Efficiency is
    time(1 GPU) / time(N GPUs) for this time-like metric (per-GPU work is fixed); the reference arm's lines, when
    given as well, add the ratio reference / ours per GPU count.
    """
    ours = sorted((r for r in records if r.get("impl", "ours") != "reference" and "value" in r), key=lambda r: r["n_gpus"])
    reference = {r["n_gpus"]: r for r in records if r.get("impl") == "reference" and "value" in r}
    if not ours:
        raise ValueError("no result line of this framework among the inputs")
    first = ours[0]
    for other in ours[1:] + list(reference.values()):
        for key in ("metric", "unit", "dtype", "higher_is_better"):
            if other.get(key) != first.get(key):
                raise ValueError(f"lines disagree on {key!r}: {first.get(key)!r} vs {other.get(key)!r}")
        for key in ("model", "seq_len"):
            if other.get("config", {}).get(key) != first.get("config", {}).get(key):
                raise ValueError(f"lines disagree on config.{key}")
    base = next((r["value"] for r in ours if r["n_gpus"] == 1), None)
    header = ["GPUs", "dispatch+combine us", "dispatch us", "combine us", "end to end us", "fraction of bound (dispatch / combine)",
              "efficiency vs 1 GPU", "reference us", "reference / ours", "payload check"]
    lines = ["| " + " | ".join(header) + " |", "|" + "---|" * len(header)]
    for r in ours:
        roof = r.get("roofline", {})
        ref = reference.get(r["n_gpus"])
        lines.append("| " + " | ".join([
            str(r["n_gpus"]), f"{r['value']:.1f}",
            f"{r['dispatch_us']:.1f}" if r.get("dispatch_us") is not None else "-",
            f"{r['combine_us']:.1f}" if r.get("combine_us") is not None else "-",
            f"{r['e2e']['value']:.1f}" if isinstance(r.get("e2e"), dict) and r["e2e"].get("value") is not None else "-",
            f"{roof.get('dispatch_fraction', float('nan')):.2f} / {roof.get('combine_fraction', float('nan')):.2f}" if roof else "-",
            f"{base / r['value']:.2f}" if base else "-",
            f"{ref['value']:.1f}" if ref else "-",
            f"{ref['value'] / r['value']:.1f}x" if ref else "-",
            payload_verdict(r),
        ]) + " |")
    return "\n".join(lines)


def payload_verdict(record: Dict) -> str:
    """What a ``bench.py`` line says about its own correctness checks: the verified exchanges before the timed loops, the
    one after them, and whether the run had to fall back to one fence per row."""
    before, after = record.get("payload_check"), record.get("payload_check_after")
    if not isinstance(before, dict):
        return "-"
    parts = ["ok" if before.get("ok") else "FAILED"]
    if isinstance(after, dict):
        parts.append("after: ok" if after.get("ok") else "after: FAILED")
    if before.get("conservative_flags"):
        parts.append("one fence per row (fallback)")
    return ", ".join(parts)


def sweep_table(record: Dict) -> str:
    """Token sweep of one ``bench.py --sweep`` line next to the reference's published dispatch latencies."""
    sweep = record.get("sweep") or {}
    if not sweep:
        raise ValueError("the line has no sweep (run bench.py with --sweep)")
    header = ["T per rank", "dispatch us", "dispatch + combine us", "published reference dispatch us (8x H20D)", "published / ours (dispatch)"]
    lines = ["| " + " | ".join(header) + " |", "|" + "---|" * len(header)]
    for tokens in sorted(sweep, key=int):
        entry = sweep[tokens]
        ref = PUBLISHED_US.get(int(tokens))
        lines.append(f"| {tokens} | {entry['dispatch_us']:.1f} | {entry['us_per_step']:.1f} | {ref if ref else '-'} | "
                     f"{ref / entry['dispatch_us']:.0f}x |" if ref else f"| {tokens} | {entry['dispatch_us']:.1f} | {entry['us_per_step']:.1f} | - | - |")
    return "\n".join(lines)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("files", type=Path, nargs="+")
    parser.add_argument("--baseline", default="", choices=["", "published"])
    parser.add_argument("--bench", action="store_true",
                        help="the files are saved outputs of bench.py (either arm, any GPU count): print the scaling table and, "
                             "for lines that carry one, the token sweep")
    args = parser.parse_args()
    if args.bench:
        records = [load_bench_line(p) for p in args.files]
        print(scaling_table(records))
        for record in records:
            if record.get("sweep"):
                print(f"\nsweep at {record['n_gpus']} GPUs\n" + sweep_table(record))
        return
    files = [load(p) for p in args.files]
    print(table(files, [p.stem for p in args.files], args.baseline))


if __name__ == "__main__":
    main()
