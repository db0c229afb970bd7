"""Runs the benchmark matrix or the acceptance groups on one node, one job after the other, and keeps what they wrote.

    python benchmarks/run_matrix.py bench --gpus 8 --rounds 2                       # the published-style sweep
    python benchmarks/run_matrix.py bench --gpus 8 --modes eager graph_cached --wires bf16 fp8_e4m3 --profiles uniform zipf
    python benchmarks/run_matrix.py bench --gpus 8 --ablation                       # plus fused against two-step dispatch
    python benchmarks/run_matrix.py validate --gpus 8 --group all
    python benchmarks/run_matrix.py bench --gpus 2 --dry-run                        # print the commands only

Every job is one subprocess (``torchrun`` for anything with more than one rank, rendezvous on 127.0.0.1) with its own
log and, where the tool writes one, its own JSON record under ``results/<run id>/``.  The run directory also gets
``manifest.json``: the source manifest of the tree (``benchmarks/source_manifest.py``), the arguments, every job's
command, exit status and duration.  Jobs never overlap: two of these programs on the same GPUs would wait for each
other's kernels.  A failing job does not stop the run; the exit status of the whole run is non-zero if any job failed.
Before a ``bench`` run NVML is asked (read-only) whether the GPUs are there and idle; busy GPUs end the run with status 3.
After a ``bench`` run the tables of ``benchmarks/report.py`` are printed from the records just written.

Parity: the reference's ``scripts/benchmark_f2.sh`` (sequential rounds with run ids, result directories, dry run)
and ``scripts/validate_f2.sh`` (acceptance groups); its container, ssh and NVLink-counter plumbing has no place here.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import time
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

RUN_ID = re.compile(r"^[A-Za-z0-9_-]+$")
TOKENS = (128, 256, 1024, 4096, 8192)
GROUPS = ("smoke", "correctness", "faults", "large", "stress", "litmus", "layer", "profiler", "path", "model", "all")


def launcher(gpus: int, port: int) -> List[str]:
    """Command prefix that starts one process per GPU (plain python for a single GPU)."""
    if gpus <= 1:
        return [sys.executable]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(gpus), "--master-addr", "127.0.0.1",
            "--master-port", str(port)]


def bench_jobs(args: argparse.Namespace, run_dir: Path) -> List[Dict]:
    jobs = []
    port = args.port
    for round_index in range(1, args.rounds + 1):
        directory = run_dir / f"round{round_index}"
        jobs.append({"name": f"round{round_index}/headline", "log": directory / "headline.log", "record": None,
                     "command": launcher(args.gpus, port) + ["bench.py", "--gpus", str(args.gpus), "--steps", str(args.steps),
                                                            "--warmup", str(args.warmup), "--sweep"]})
        port += 1
        for mode in args.modes:
            for wire in args.wires:
                for profile in args.profiles:
                    name = f"{mode}_{wire}_{profile}"
                    record = directory / f"{name}.json"
                    command = launcher(args.gpus, port) + ["benchmarks/benchmark.py", "--tokens", *map(str, args.tokens), "--mode", mode,
                                                           "--wire", wire, "--profile", profile, "--iterations", str(args.iterations),
                                                           "--output", str(record)]
                    if profile != "uniform":
                        command += ["--topk", "4"]  # the frozen non-uniform fixtures are top-4
                    jobs.append({"name": f"round{round_index}/{name}", "log": directory / f"{name}.log", "record": record, "command": command})
                    port += 1
        if args.ablation:
            jobs.append({"name": f"round{round_index}/ablation_unfused", "log": directory / "ablation_unfused.log", "record": None,
                         "command": launcher(args.gpus, port) + ["benchmarks/ablation_unfused.py", "--tokens", *map(str, args.tokens),
                                                                "--iterations", str(args.iterations)]})
            port += 1
        if args.nccl and args.gpus > 1:
            jobs.append({"name": f"round{round_index}/nccl", "log": directory / "nccl.log", "record": None,
                         "command": launcher(args.gpus, port) + ["benchmarks/benchmark_nccl.py", "--tokens", *map(str, args.tokens)]})
            port += 1
    return jobs


def validate_jobs(args: argparse.Namespace, run_dir: Path) -> List[Dict]:
    groups = [g for g in GROUPS if g != "all"] if args.group == "all" else [args.group]
    pytest = [sys.executable, "-m", "pytest", "-q", "-x"]
    jobs = []
    port = args.port
    for group in groups:
        if group == "smoke":
            command = [sys.executable, "-c", "import __graft_entry__ as g; g.smoke(); print('smoke ok')"]
        elif group == "correctness":
            command = pytest + ["-m", "gpu", "tests/test_gpu_dispatch.py", "tests/test_gpu_api.py", "tests/test_gpu_scale.py",
                                "tests/test_gpu_multiprocess.py", "tests/test_zz_no_alloc.py"]
        elif group == "faults":
            command = pytest + ["-m", "gpu", "tests/test_gpu_faults.py"]
        elif group == "large":
            command = launcher(args.gpus, port) + ["tests/workers/ep_worker.py", "--transport", "peer", "--suite", "large", "--tokens",
                                                   "4096,8192", "--timeout-ms", "20000"]
        elif group == "stress":
            command = pytest + ["-m", "gpu", "tests/test_gpu_scale.py", "-k", "epochs"]
        elif group == "litmus":
            command = pytest + ["-m", "gpu", "tests/test_gpu_litmus.py"]
        elif group == "layer":
            command = pytest + ["-m", "gpu", "tests/test_gpu_gemm.py", "tests/test_gpu_fused_combine.py"]
        elif group == "profiler":
            command = [sys.executable, "benchmarks/analysis_dispatch_profile.py", "--collect", str(run_dir / group / "trace.json"), "--tokens", "1024"]
        elif group == "path":  # NVLink counters against the deduplicated route volume (needs two GPUs or more)
            command = launcher(args.gpus, port) + ["benchmarks/nvlink_audit.py", "--tokens", "4096"]
        else:  # model: the host model of the protocol, also under ThreadSanitizer (no GPU)
            command = pytest + ["tests/test_protocol_model.py"]
        job = {"name": group, "log": run_dir / group / "log.txt", "record": None, "command": command}
        if group == "stress":
            job["env"] = {"PCIE_EP_B200_STRESS_EPOCHS": str(args.stress_epochs)}
        jobs.append(job)
        port += 1
    return jobs


def preflight(gpus: int, nvml: object = None) -> List[str]:
    """Reasons not to benchmark now: GPUs that are missing or already busy.  Only reads (NVML queries); never changes a
    clock, a power limit or any other setting of a GPU."""
    try:
        if nvml is None:
            import pynvml as nvml  # type: ignore[no-redef]
        nvml.nvmlInit()
    except Exception as exc:  # noqa: BLE001 - no NVML: nothing to check against
        return [f"NVML is not available ({type(exc).__name__}): the GPUs' state is unknown"]
    problems = []
    try:
        count = nvml.nvmlDeviceGetCount()
        if count < gpus:
            problems.append(f"{gpus} GPUs wanted, {count} present")
        for index in range(min(gpus, count)):
            handle = nvml.nvmlDeviceGetHandleByIndex(index)
            processes = nvml.nvmlDeviceGetComputeRunningProcesses(handle)
            busy = nvml.nvmlDeviceGetUtilizationRates(handle).gpu
            if processes:
                problems.append(f"GPU {index}: {len(processes)} compute process(es) already running")
            elif busy > 10:
                problems.append(f"GPU {index}: {busy} % busy")
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:  # noqa: BLE001
            pass
    return problems


def execute(job: Dict) -> int:
    job["log"].parent.mkdir(parents=True, exist_ok=True)
    with open(job["log"], "w") as log:
        return subprocess.run(job["command"], cwd=str(ROOT), stdout=log, stderr=subprocess.STDOUT,
                              env=dict(os.environ, **job.get("env", {}))).returncode


def run(args: argparse.Namespace, runner: Callable[[Dict], int] = execute) -> int:
    run_id = args.run_id or f"{args.what}_{time.strftime('%Y%m%dT%H%M%SZ', time.gmtime())}_{os.getpid()}"
    if not RUN_ID.match(run_id):
        raise SystemExit("a run id may contain only letters, digits, underscore and hyphen")
    run_dir = Path(args.results) / run_id
    jobs = bench_jobs(args, run_dir) if args.what == "bench" else validate_jobs(args, run_dir)
    if args.dry_run:
        for job in jobs:
            print(job["name"] + ": " + " ".join(job["command"]))
        return 0
    if args.what == "bench" and args.preflight:
        problems = preflight(args.gpus)
        if problems:
            print("not benchmarking: " + "; ".join(problems) + "  (--no-preflight runs anyway)", file=sys.stderr)
            return 3
    run_dir.mkdir(parents=True, exist_ok=True)
    from benchmarks import source_manifest

    manifest = {"run_id": run_id, "what": args.what, "arguments": {k: (str(v) if isinstance(v, Path) else v) for k, v in vars(args).items()},
                "sources": source_manifest.manifest(), "jobs": []}
    failed = 0
    for job in jobs:
        started = time.time()
        status = runner(job)
        manifest["jobs"].append({"name": job["name"], "command": job["command"], "exit": status, "seconds": round(time.time() - started, 1),
                                 "log": str(job["log"]), "record": str(job["record"]) if job["record"] else None})
        failed += status != 0
        print(f"[{'ok' if status == 0 else 'FAILED ' + str(status)}] {job['name']}  ({manifest['jobs'][-1]['seconds']} s)", flush=True)
        (run_dir / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    if args.what == "bench":
        print_tables(manifest)
    return 1 if failed else 0


def print_tables(manifest: Dict) -> None:
    """Tables of benchmarks/report.py from what the run wrote (jobs that failed are left out)."""
    from benchmarks import report

    headlines = [Path(j["log"]) for j in manifest["jobs"] if j["name"].endswith("/headline") and j["exit"] == 0]
    lines = []
    for path in headlines:
        try:
            lines.append(report.load_bench_line(path))
        except ValueError:
            pass
    if lines:
        print(report.scaling_table(lines[-1:]))
        if lines[-1].get("sweep"):
            print(report.sweep_table(lines[-1]))
    for job in manifest["jobs"]:
        if job["record"] and job["exit"] == 0 and Path(job["record"]).exists():
            print(f"\n{job['name']}")
            print(report.table([report.load(Path(job["record"]))], [Path(job["record"]).stem], "published" if "_uniform" in job["name"] else ""))


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = parser.add_subparsers(dest="what", required=True)
    for name in ("bench", "validate"):
        p = sub.add_parser(name)
        p.add_argument("--gpus", type=int, default=1)
        p.add_argument("--results", type=Path, default=ROOT / "results")
        p.add_argument("--run-id", default="")
        p.add_argument("--port", type=int, default=29600)
        p.add_argument("--dry-run", action="store_true")
        if name == "bench":
            p.add_argument("--rounds", type=int, default=2)
            p.add_argument("--steps", type=int, default=20)
            p.add_argument("--warmup", type=int, default=5)
            p.add_argument("--iterations", type=int, default=20)
            p.add_argument("--tokens", type=int, nargs="+", default=list(TOKENS))
            p.add_argument("--modes", nargs="+", default=["eager"], choices=["eager", "cached", "graph", "graph_cached"])
            p.add_argument("--wires", nargs="+", default=["bf16"], choices=["bf16", "fp8_e4m3"])
            p.add_argument("--profiles", nargs="+", default=["uniform"], choices=["uniform", "hotspot_20_80", "zipf", "nvidia_calibrated"])
            p.add_argument("--no-nccl", dest="nccl", action="store_false")
            p.add_argument("--ablation", action="store_true", help="also time the two-step form (unique rows, then a separate scatter pass)")
            p.add_argument("--no-preflight", dest="preflight", action="store_false",
                           help="benchmark even if NVML shows other compute processes or load on the GPUs")
        else:
            p.add_argument("--group", default="smoke", choices=GROUPS)
            p.add_argument("--stress-epochs", type=int, default=100000, help="back-to-back epochs of the stress group")
    return parser


def main(argv: Optional[Sequence[str]] = None) -> int:
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    raise SystemExit(main())
