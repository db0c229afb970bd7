"""The documents name files that exist: every path of this repository that README, DESIGN, API, BASELINE or a profile
summary puts in backticks is checked (paths of the reference, which the documents also cite, are listed below)."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
DOCUMENTS = ["README.md", "DESIGN.md", "API.md", "BASELINE.md"] + [str(p.relative_to(ROOT)) for p in sorted((ROOT / "profiles").glob("*.md"))]
PREFIXES = ("pcie_ep_b200/", "csrc/", "benchmarks/", "tests/", "profiles/", "examples/")
# files of the reference that the documents cite by the same kind of path
REFERENCE_ONLY = {"benchmarks/benchmark_nccl_shm.py", "benchmarks/data/control_progress_profile.json", "benchmarks/data/nccl_shm_c32_comparison.md",
                  "csrc/runtime.cu", "benchmarks/csrc/nccl_expand.cu", "tests/test_large.py", "tests/mapped_litmus.cu", "tests/MAPPED_LITMUS.md"}


def cited_paths(text):
    for found in re.findall(r"`([A-Za-z0-9_./{},*-]+\.(?:py|cu|cuh|hpp|cpp|h|md|json|npz))`", text):
        if "*" in found:
            continue
        if "{" in found:
            head, rest = found.split("{", 1)
            alternatives, tail = rest.split("}", 1)
            yield from (head + a + tail for a in alternatives.split(","))
        else:
            yield found


def test_every_cited_file_of_this_repository_exists():
    missing = []
    for document in DOCUMENTS:
        for path in cited_paths((ROOT / document).read_text()):
            if not path.startswith(PREFIXES) or path in REFERENCE_ONLY:
                continue
            if not (ROOT / path).exists():
                missing.append(f"{document}: {path}")
    assert not missing, missing
