"""Provenance of a result: which sources and flags the native library was built from, plus a source-level audit.

    python benchmarks/source_manifest.py                       # print the manifest of this tree as JSON
    python benchmarks/source_manifest.py --output manifest.json
    python benchmarks/source_manifest.py --check manifest.json # does the tree still match a saved manifest?
    python benchmarks/source_manifest.py --audit               # source rules of the protocol (exit 1 on a violation)

The manifest lists every file the extension is compiled from with its SHA-256, the compiler flags, the combined
fingerprint (the same value the loader stamps next to the built library, so "was this number measured with these
sources" has a yes/no answer) and the toolchain versions.  ``bench.py`` and ``benchmarks/benchmark.py`` put the
fingerprint into their records.

The audit reads the kernels as text and checks the rules the protocol relies on:

* read-modify-write operations only ever address memory of the issuing GPU (counters, statistics, error words):
  the segment of a peer is only written with plain stores and only polled locally, so no atomic may take an
  address formed from the peer table;
* every loop that polls a flag or an mbarrier carries a deadline (a bounded wait that records an error code);
* no load with cluster multicast and none of the batched copy calls that this library never uses;
* the Python launch path (dispatch, combine, the fused launch, graph replay, the stream policy) calls nothing that
  makes the host wait for the device or reads device memory back (`.item()`, `.cpu()`, `.tolist()`, `synchronize`, ...).

Parity: the reference's ``scripts/source_manifest.py`` and the read-modify-write provenance part of its
``scripts/collect_advanced_path_audit.py`` (its machine-code dump is not reproduced).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import re
import sys
from pathlib import Path
from typing import Dict, List

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

NATIVE_SUFFIXES = (".cu", ".cuh", ".cpp", ".hpp", ".h")
ATOMIC_CALL = re.compile(r"\b(atomic(?:Add|Sub|Exch|CAS|Min|Max|Or|And|Xor|Inc|Dec))\s*\(\s*([^,]+),")
ATOMIC_PTX = re.compile(r"\b(atom|red)\.(?:[a-z_0-9:.]+)")
PEER_ADDRESS = re.compile(r"seg\s*\[|peer_|remote_|dst_of|->seg\b")
POLL_LOOP = re.compile(r"\bwhile\s*\(.*(ld_acquire_|ld_relaxed_|ld_volatile|try_wait|mbar_test)")
BOUND_WORDS = ("give_up(", "deadline", "expired", "timed_out", "spins", "polls", "budget")
LOOP_WINDOW = 10
# assembled from pieces so that this file does not itself contain the names it looks for
FORBIDDEN = {
    "load with cluster multicast": re.compile(r"cp\.async\.bulk[a-z0-9_.:]*" + re.escape(".multi" + "cast::cluster")),
    "batched copy call": re.compile(r"\bcu(?:da)?Memcpy(?:3D)?" + "Batch" + r"Async\b"),
}


def native_files(root: Path = ROOT) -> List[Path]:
    return sorted(p for p in (root / "csrc").rglob("*") if p.suffix in NATIVE_SUFFIXES)


def manifest(root: Path = ROOT) -> Dict:
    from pcie_ep_b200 import _C

    files = {str(p.relative_to(root)): hashlib.sha256(p.read_bytes()).hexdigest() for p in native_files(root)}
    versions = {}
    try:
        import torch

        versions = {"torch": torch.__version__, "cuda": torch.version.cuda}
    except ImportError:
        pass
    return {
        "fingerprint": _C.source_fingerprint(),
        "library_matches_sources": _C.is_built(),
        "cuda_flags": list(_C.CUDA_FLAGS),
        "host_flags": list(_C.HOST_FLAGS),
        "translation_units": [str(p.relative_to(root)) for p in _C.SOURCES],
        "files": files,
        "versions": versions,
    }


def compare(saved: Dict, current: Dict) -> List[str]:
    """Human-readable differences between a saved manifest and the tree (empty list = identical sources and flags)."""
    out = []
    for key in ("cuda_flags", "host_flags"):
        if saved.get(key) != current.get(key):
            out.append(f"{key} changed: {saved.get(key)} -> {current.get(key)}")
    old, new = saved.get("files", {}), current.get("files", {})
    for name in sorted(set(old) | set(new)):
        if name not in new:
            out.append(f"removed: {name}")
        elif name not in old:
            out.append(f"added: {name}")
        elif old[name] != new[name]:
            out.append(f"modified: {name}")
    if not out and saved.get("fingerprint") != current.get("fingerprint"):
        out.append("fingerprint differs although no listed file does")
    return out


def strip_comments(text: str) -> str:
    """Blank out // and /* */ comments, keeping line numbers."""
    text = re.sub(r"/\*.*?\*/", lambda m: re.sub(r"[^\n]", " ", m.group(0)), text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def audit_text(name: str, text: str) -> Dict[str, List[str]]:
    """{"atomics": [...every read-modify-write with its target...], "violations": [...]} for one source text."""
    atomics, violations = [], []
    lines = strip_comments(text).splitlines()
    for number, line in enumerate(lines, 1):
        for match in ATOMIC_CALL.finditer(line):
            target = match.group(2).strip()
            atomics.append(f"{name}:{number}: {match.group(1)} on {target}")
            if PEER_ADDRESS.search(target):
                violations.append(f"{name}:{number}: {match.group(1)} addresses peer memory ({target})")
        if "asm" in line and ATOMIC_PTX.search(line):
            atomics.append(f"{name}:{number}: inline {ATOMIC_PTX.search(line).group(0)}")
            if PEER_ADDRESS.search(line):
                violations.append(f"{name}:{number}: inline read-modify-write next to a peer address")
        for label, pattern in FORBIDDEN.items():
            if pattern.search(line):
                violations.append(f"{name}:{number}: {label}")
        if POLL_LOOP.search(line):
            window = " ".join(lines[number - 1:number - 1 + LOOP_WINDOW])
            if not any(word in window for word in BOUND_WORDS):
                violations.append(f"{name}:{number}: polling loop without a deadline in its first {LOOP_WINDOW} lines")
    return {"atomics": atomics, "violations": violations}


# Calls that make the host wait for the device or read device memory back.  The launch path (dispatch, combine, the
# fused launch, a graph replay and what they go through) must contain none: sizes stay on the device, errors are only
# read by check_errors().
HOST_WAITING_CALLS = ("item", "cpu", "tolist", "numpy", "synchronize")
HOT_PATH = {
    "pcie_ep_b200/buffers/ep.py": ("dispatch", "combine", "fused_expert_combine", "_enqueue", "capture_dispatch"),
    "pcie_ep_b200/graph.py": ("replay",),
    "pcie_ep_b200/buffers/streams.py": ("begin", "finish", "current"),
}


def audit_python(name: str, text: str, functions: tuple) -> List[str]:
    """Host-waiting calls inside the named functions of one Python source (nested helpers included)."""
    import ast

    found = []
    tree = ast.parse(text)
    for node in ast.walk(tree):
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and node.name in functions:
            for inner in ast.walk(node):
                if isinstance(inner, ast.Call) and isinstance(inner.func, ast.Attribute) and inner.func.attr in HOST_WAITING_CALLS:
                    found.append(f"{name}:{inner.lineno}: {node.name}() calls .{inner.func.attr}()")
    return found


def audit(root: Path = ROOT) -> Dict[str, List[str]]:
    result: Dict[str, List[str]] = {"atomics": [], "violations": []}
    for path in native_files(root):
        part = audit_text(str(path.relative_to(root)), path.read_text())
        result["atomics"] += part["atomics"]
        result["violations"] += part["violations"]
    for name, functions in HOT_PATH.items():
        path = root / name
        if path.exists():
            result["violations"] += audit_python(name, path.read_text(), functions)
    return result


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--output", type=Path)
    parser.add_argument("--check", type=Path, help="saved manifest to compare the tree with")
    parser.add_argument("--audit", action="store_true")
    args = parser.parse_args()
    if args.audit:
        result = audit()
        print(f"{len(result['atomics'])} read-modify-write sites, all on local memory" if not result["violations"]
              else "\n".join(result["violations"]))
        raise SystemExit(1 if result["violations"] else 0)
    current = manifest()
    if args.check:
        differences = compare(json.loads(args.check.read_text()), current)
        print("identical" if not differences else "\n".join(differences))
        raise SystemExit(1 if differences else 0)
    text = json.dumps(current, indent=2)
    if args.output:
        args.output.write_text(text + "\n")
    else:
        print(text)


if __name__ == "__main__":
    main()
