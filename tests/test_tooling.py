"""Benchmark tooling that runs without a GPU: report recomputation and footprint arithmetic
(reference: tests/test_report_latest.py, test_report_control_progress.py, RESULTS_HOST_BUFFER.md)."""

import json

import pytest

from benchmarks import report
from benchmarks.memory_footprint import footprint


def _record_file(tmp_path, name, world=8, profile="uniform", dispatch=(100.0, 500.0)):
    data = {"arguments": {"hidden": "7168", "experts": "256", "topk": "8", "profile": profile, "wire": "bf16"},
            "records": [{"tokens": t, "world": world, "dispatch_us_mean": d, "combine_us_mean": d * 1.1}
                        for t, d in zip((128, 4096), dispatch)]}
    path = tmp_path / f"{name}.json"
    path.write_text(json.dumps(data))
    return path


def test_report_table_and_published_baseline(tmp_path):
    a = _record_file(tmp_path, "eager")
    b = _record_file(tmp_path, "graph", dispatch=(60.0, 480.0))
    text = report.table([report.load(a), report.load(b)], ["eager", "graph"], "published")
    assert "| 128 | 100.0 | 60.0 |" in text and "647" in text and "6.5x" in text
    assert "| 4096 | 500.0 | 480.0 |" in text and "27.1x" in text


def test_report_refuses_mixed_configurations(tmp_path):
    a = _record_file(tmp_path, "a")
    with pytest.raises(ValueError, match="profile"):
        report.table([report.load(a), report.load(_record_file(tmp_path, "b", profile="zipf"))], ["a", "b"])
    with pytest.raises(ValueError, match="world"):
        report.table([report.load(a), report.load(_record_file(tmp_path, "c", world=4))], ["a", "c"])
    bad = tmp_path / "bad.json"
    bad.write_text("{}")
    with pytest.raises(ValueError):
        report.load(bad)


def test_footprint_arithmetic(ext):
    f = footprint(8, 8192, 7168, 8, 256, 32, 0, 3, False, True, False)
    assert f["row_stride"] == 14464 and f["slots"] == 256
    assert f["segment_staging_bytes"] == 8 * 32 * 256 * 14464
    assert f["expanded_capacity_rows"] == 8 * 8192 * 8 + 32 * 255
    assert f["segment_bytes"] >= f["segment_staging_bytes"] + f["segment_combine_bytes"]
    relay = footprint(8, 8192, 7168, 8, 256, 32, 0, 3, False, True, True)
    assert relay["outboxes_bytes"] == 7 * relay["segment_bytes"]
    bounded = footprint(8, 8192, 7168, 8, 256, 32, 16, 3, False, False, False)
    assert bounded["slots"] == 16 and bounded["segment_bytes"] < f["segment_bytes"] // 8


def test_bench_routes_and_roofline_model():
    """The headline benchmark's synthetic routing is deterministic per (rank, tokens) and its roofline is the slower
    of the HBM and the NVLink bound: HBM-bound at one rank, NVLink-bound at eight."""
    import torch

    import bench

    idx_a, w_a = bench.make_routes(256, 256, 8, rank=3)
    idx_b, w_b = bench.make_routes(256, 256, 8, rank=3)
    assert torch.equal(idx_a, idx_b) and torch.equal(w_a, w_b)
    assert not torch.equal(idx_a, bench.make_routes(256, 256, 8, rank=4)[0])
    assert all(len(set(row)) == 8 for row in idx_a.tolist())  # distinct experts per token
    assert torch.allclose(w_a.sum(dim=1), torch.ones(256))
    one = bench.roofline(idx_a, 1, 0, 256, 8, 256)
    eight = bench.roofline(idx_a, 8, 3, 256, 8, 256)
    assert one["dispatch_bound"] == "hbm" and one["combine_bound"] == "hbm"
    assert eight["dispatch_bound"] == "nvlink" and eight["combine_bound"] == "nvlink"
    assert eight["dispatch_us"] > one["dispatch_us"] > 0
    # one rank, BF16: x read + expanded rows written = (1 + 8) * 256 rows of 14,336 bytes at the copy rate
    assert abs(one["dispatch_us"] - 9 * 256 * 14336 / 6548e9 * 1e6) / one["dispatch_us"] < 0.05


def _trace(extra=()):
    """A hand-made Chrome trace: two markers, launches inside and outside them, kernels linked by correlation id."""
    events = [
        {"ph": "X", "cat": "user_annotation", "name": "ep.dispatch", "ts": 100, "dur": 50, "tid": 1},
        {"ph": "X", "cat": "user_annotation", "name": "ep.combine", "ts": 200, "dur": 60, "tid": 1},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernelExC", "ts": 110, "dur": 5, "tid": 1, "args": {"correlation": 1}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": 210, "dur": 5, "tid": 1, "args": {"correlation": 2}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": 230, "dur": 5, "tid": 1, "args": {"correlation": 3}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": 400, "dur": 5, "tid": 1, "args": {"correlation": 4}},
        # kernels run later than their launches, possibly after the marker has ended on the host
        {"ph": "X", "cat": "kernel", "name": "bep::dispatch_kernel(bep::DispatchLaunch)", "ts": 160, "dur": 140, "args": {"correlation": 1}},
        {"ph": "X", "cat": "kernel", "name": "bep::combine_push_kernel(bep::CombinePushArgs)", "ts": 310, "dur": 90, "args": {"correlation": 2}},
        {"ph": "X", "cat": "kernel", "name": "bep::fused_reduce_kernel(bep::FusedReduceArgs)", "ts": 405, "dur": 30, "args": {"correlation": 3}},
        {"ph": "X", "cat": "kernel", "name": "elementwise_kernel", "ts": 500, "dur": 3, "args": {"correlation": 4}},
    ]
    return {"traceEvents": events + list(extra)}


def test_trace_attribution_by_correlation_id():
    from benchmarks.analysis_dispatch_profile import attribute, audit, format_report

    report = attribute(_trace())
    assert [k for k, _ in report["ep.dispatch"]["kernels"]] == ["bep::dispatch_kernel(bep::DispatchLaunch)"]
    assert len(report["ep.combine"]["kernels"]) == 2 and report["ep.combine"]["device_us"] == 120
    assert [k for k, _ in report["(outside)"]["kernels"]] == ["elementwise_kernel"]
    assert audit(report) == []
    assert "dispatch_kernel" in format_report(report)


def test_trace_audit_flags_nccl_sync_and_readback():
    from benchmarks.analysis_dispatch_profile import attribute, audit

    bad = _trace([
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": 120, "dur": 2, "tid": 1, "args": {"correlation": 9}},
        {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllGather_RING_LL", "ts": 300, "dur": 50, "args": {"correlation": 9}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaStreamSynchronize", "ts": 130, "dur": 20, "tid": 1, "args": {"correlation": 10}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaMemcpyAsync", "ts": 240, "dur": 2, "tid": 1, "args": {"correlation": 11}},
        {"ph": "X", "cat": "gpu_memcpy", "name": "Memcpy DtoH (Device -> Pinned)", "ts": 420, "dur": 2, "args": {"correlation": 11}},
    ])
    problems = audit(attribute(bad))
    assert any("NCCL" in p for p in problems) and any("cudaStreamSynchronize" in p for p in problems)
    assert any("device-to-host" in p for p in problems) and len(problems) == 3


def test_role_summary_layouts():
    import torch

    from benchmarks.analysis_dispatch_profile import summarise_roles

    assert summarise_roles(torch.zeros(0, 16, 16), 4, 2, 2, 3) == {}
    role = torch.zeros(6, 16, 16)
    role[4:6, 0:2, 0] = 10     # two sender CTAs, two send warps each: 10 rows per warp
    role[0:4, 1:4, 0] = 5      # four channel CTAs, three receive warps each
    role[0:4, 1:4, 8] = 2
    summary = summarise_roles(role, channels=4, send_ctas=2, tx_warps=2, rx_warps=3)
    assert summary["send"]["rows"] == 10 and summary["send"]["warps"] == 4
    assert summary["receive"]["rows"] == 5 and summary["receive"]["local_rows"] == 2 and summary["receive"]["warps"] == 12
    inside = torch.zeros(4, 16, 16)
    inside[:, 1:3, 0] = 7
    inside[:, 3:6, 0] = 3
    summary = summarise_roles(inside, channels=4, send_ctas=0, tx_warps=2, rx_warps=3)
    assert summary["send"]["rows"] == 7 and summary["receive"]["rows"] == 3


def test_smaps_rollup_parser():
    from benchmarks.memory_footprint import parse_smaps_rollup

    text = ("55d0c0a00000-7ffd1c5f2000 ---p 00000000 00:00 0                          [rollup]\n"
            "Rss:              123456 kB\nPss:               65432 kB\nPss_Shmem:         2048 kB\nSwap:                  0 kB\n")
    counters = parse_smaps_rollup(text)
    assert counters == {"Rss": 123456 * 1024, "Pss": 65432 * 1024, "Pss_Shmem": 2048 * 1024, "Swap": 0}


def _bench_line(n_gpus, value, impl="ours", **extra):
    line = {"metric": "dispatch+combine us", "value": value, "unit": "us/step", "n_gpus": n_gpus, "dtype": "bf16",
            "higher_is_better": False, "impl": impl, "config": {"model": "moe-dispatch", "seq_len": 4096},
            "dispatch_us": value * 0.45, "combine_us": value * 0.55, "e2e": {"value": value + 800.0},
            "roofline": {"dispatch_fraction": 0.6, "combine_fraction": 0.5}}
    line.update(extra)
    return line


def test_scaling_table_from_bench_lines(tmp_path):
    paths = []
    for n, v, impl in ((1, 200.0, "ours"), (2, 400.0, "ours"), (2, 4000.0, "reference")):
        path = tmp_path / f"{impl}{n}.log"
        path.write_text("some log line\n" + json.dumps(_bench_line(n, v, impl)) + "\n")
        paths.append(path)
    text = report.scaling_table([report.load_bench_line(p) for p in paths])
    rows = [r for r in text.splitlines() if r.startswith("| 2 ")]
    assert len(rows) == 1 and "0.50" in rows[0] and "10.0x" in rows[0] and "4000.0" in rows[0]
    assert "| 1 | 200.0" in text and "1.00" in text


def test_scaling_table_refuses_lines_of_different_metrics():
    other = _bench_line(2, 300.0)
    other["metric"] = "dispatch us"
    with pytest.raises(ValueError, match="metric"):
        report.scaling_table([_bench_line(1, 200.0), other])
    with pytest.raises(ValueError, match="no result line"):
        report.scaling_table([_bench_line(1, 1.0, impl="reference")])


def test_sweep_table_uses_published_numbers():
    line = _bench_line(8, 900.0, sweep={"128": {"dispatch_us": 64.7, "us_per_step": 120.0}, "4096": {"dispatch_us": 400.0, "us_per_step": 900.0}})
    text = report.sweep_table(line)
    assert "| 128 | 64.7 | 120.0 | 647 | 10x |" in text and "| 4096 | 400.0 | 900.0 | 13558 | 34x |" in text


def test_committed_bench_samples_recompute():
    from pathlib import Path

    samples = sorted((Path(report.__file__).parent / "data" / "results").glob("bench_*gpu*.json"))
    assert samples, "sample results are part of the repository"
    text = report.scaling_table([report.load_bench_line(p) for p in samples])
    assert text.count("\n") >= 2


def test_source_audit_is_clean_and_sees_violations():
    from benchmarks import source_manifest

    result = source_manifest.audit()
    assert result["violations"] == []
    assert len(result["atomics"]) > 20
    bad = source_manifest.audit_text("x.cu", "void f() {\n  atomicAdd(rc->seg[p] + 4, 1);\n  while (ptx::ld_acquire_sys(flag) != v) {\n    ++n;\n  }\n}\n")
    assert len(bad["violations"]) == 2
    assert "peer memory" in bad["violations"][0] and "polling loop" in bad["violations"][1]
    commented = source_manifest.audit_text("x.cu", "// atomicAdd(rc->seg[p], 1);\n/* while (ptx::ld_acquire_sys(f)) {} */\n")
    assert commented["violations"] == [] and commented["atomics"] == []


def test_source_manifest_compare(ext):
    from benchmarks import source_manifest

    current = source_manifest.manifest()
    assert current["fingerprint"] and "csrc/kernels/dispatch.cuh" in current["files"]
    assert source_manifest.compare(current, current) == []
    changed = json.loads(json.dumps(current))
    changed["files"]["csrc/kernels/dispatch.cuh"] = "0" * 64
    changed["files"].pop("csrc/kernels/ptx.cuh")
    changed["cuda_flags"] = ["-O0"]
    differences = source_manifest.compare(changed, current)
    assert any(d.startswith("modified: csrc/kernels/dispatch.cuh") for d in differences)
    assert any(d.startswith("added: csrc/kernels/ptx.cuh") for d in differences) and any("cuda_flags" in d for d in differences)


def test_run_matrix_plans_sequential_jobs_and_records_them(tmp_path):
    from benchmarks import run_matrix

    parser = run_matrix.build_parser()
    args = parser.parse_args(["bench", "--gpus", "4", "--rounds", "2", "--modes", "eager", "graph_cached", "--wires", "bf16", "fp8_e4m3",
                              "--profiles", "uniform", "zipf", "--results", str(tmp_path), "--run-id", "unit_1"])
    jobs = run_matrix.bench_jobs(args, tmp_path / "unit_1")
    assert len(jobs) == 2 * (1 + 2 * 2 * 2 + 1)                       # headline + matrix + NCCL comparison, per round
    ports = [j["command"][j["command"].index("--master-port") + 1] for j in jobs]
    assert len(set(ports)) == len(ports)                               # no two jobs share a rendezvous port
    assert all("--master-addr" in j["command"] and "127.0.0.1" in j["command"] for j in jobs)
    with_ablation = run_matrix.bench_jobs(parser.parse_args(["bench", "--gpus", "4", "--rounds", "1", "--ablation"]), tmp_path / "unit_2")
    assert sum("benchmarks/ablation_unfused.py" in j["command"] for j in with_ablation) == 1   # once per round, only on request
    assert not any("benchmarks/ablation_unfused.py" in j["command"] for j in jobs)
    zipf = [j for j in jobs if j["name"].endswith("eager_bf16_zipf")][0]
    assert zipf["command"][-2:] == ["--topk", "4"] and str(zipf["record"]).endswith("eager_bf16_zipf.json")

    ran = []

    def fake(job):
        ran.append(job["name"])
        job["log"].parent.mkdir(parents=True, exist_ok=True)
        job["log"].write_text("")
        return 3 if job["name"].endswith("nccl") else 0

    args.preflight = False
    assert run_matrix.run(args, runner=fake) == 1                      # a failed job fails the run, but every job still ran
    assert ran == [j["name"] for j in jobs]
    manifest = json.loads((tmp_path / "unit_1" / "manifest.json").read_text())
    assert [j["exit"] for j in manifest["jobs"]].count(3) == 2 and manifest["sources"]["fingerprint"]

    with pytest.raises(SystemExit):
        run_matrix.run(parser.parse_args(["bench", "--run-id", "bad id", "--results", str(tmp_path)]), runner=fake)
    single = run_matrix.validate_jobs(parser.parse_args(["validate", "--group", "all", "--gpus", "1"]), tmp_path / "v")
    assert [j["name"] for j in single] == [g for g in run_matrix.GROUPS if g != "all"]
    assert single[3]["command"][0].endswith("python") or "python" in single[3]["command"][0]   # one GPU: no torchrun
    assert "torch.distributed.run" not in single[3]["command"]


def test_preflight_only_reads_and_names_busy_gpus():
    from types import SimpleNamespace

    from benchmarks import run_matrix

    calls = []

    class FakeNvml:
        def __init__(self, processes, busy):
            self.processes, self.busy = processes, busy

        def __getattr__(self, name):
            calls.append(name)
            table = {
                "nvmlInit": lambda: None, "nvmlShutdown": lambda: None, "nvmlDeviceGetCount": lambda: 2,
                "nvmlDeviceGetHandleByIndex": lambda i: i,
                "nvmlDeviceGetComputeRunningProcesses": lambda h: self.processes[h],
                "nvmlDeviceGetUtilizationRates": lambda h: SimpleNamespace(gpu=self.busy[h]),
            }
            return table[name]

    assert run_matrix.preflight(2, FakeNvml([[], []], [0, 3])) == []
    problems = run_matrix.preflight(4, FakeNvml([[1], []], [0, 55]))
    assert problems == ["4 GPUs wanted, 2 present", "GPU 0: 1 compute process(es) already running", "GPU 1: 55 % busy"]
    assert all(name.startswith(("nvmlInit", "nvmlShutdown", "nvmlDeviceGet")) for name in calls)   # queries only, no setters


def test_python_launch_path_audit_sees_host_waits():
    from benchmarks import source_manifest

    bad = "class B:\n    def dispatch(self, x):\n        n = x.sum().item()\n        def inner():\n            torch.cuda.synchronize()\n        return n\n    def other(self, x):\n        return x.cpu()\n"
    found = source_manifest.audit_python("b.py", bad, ("dispatch",))
    assert len(found) == 2 and ".item()" in found[0] and ".synchronize()" in found[1]
    assert source_manifest.audit()["violations"] == []


def test_bench_repeated_check_keeps_ranks_in_step_and_stops_at_the_first_bad_round():
    import bench

    calls = {"verify": 0, "gather": 0}

    def gather_two(out, mine):               # the other rank always agrees with this one
        calls["gather"] += 1
        out[0], out[1] = mine, dict(mine)

    def fine():
        calls["verify"] += 1
        return {"ok": True, "rows_checked": 4, "elements_checked": 8, "problems": []}

    verdict, everyone, ok = bench.repeated_check(fine, gather_two, 2, rounds=3)
    assert ok and calls == {"verify": 3, "gather": 3} and len(everyone) == 2 and verdict["rows_checked"] == 4

    sequence = iter([True, False, True])

    def second_round_bad():
        if next(sequence):
            return {"ok": True, "rows_checked": 1, "elements_checked": 1, "problems": []}
        raise RuntimeError("EP dispatch GPU error on rank 1: [18, 0, 3]")

    calls["gather"] = 0
    verdict, everyone, ok = bench.repeated_check(second_round_bad, gather_two, 2, rounds=3)
    assert not ok and calls["gather"] == 2                       # the failing round is still gathered, the third never runs
    assert verdict["ok"] is False and "GPU error" in verdict["problems"][0]

    def peer_bad(out, mine):                 # this rank is fine, the other one is not
        out[0], out[1] = mine, {"ok": False, "rows_checked": 0, "elements_checked": 0, "problems": ["rows 0..4096 differ"]}

    verdict, everyone, ok = bench.repeated_check(fine, peer_bad, 2, rounds=3)
    assert not ok and verdict["ok"] is True and everyone[1]["problems"] == ["rows 0..4096 differ"]


def test_bench_falls_back_to_the_conservative_publication_once_and_says_so():
    import bench

    class FakeBuffer:
        built = 0

        def __init__(self, env):
            FakeBuffer.built += 1
            self.conservative = env.get(bench.FENCE_ENV) == "1"   # the runtime reads the setting when it is built
            self.closed = False

        def close(self):
            self.closed = True
            raise RuntimeError("a failed buffer may refuse an orderly close")

    def check(buffer):
        good = {"ok": True, "rows_checked": 5, "elements_checked": 50, "problems": []}
        bad = {"ok": False, "rows_checked": 0, "elements_checked": 0, "problems": ["rows 0..4096 differ from their source"]}
        return (good, [good, good], True) if buffer.conservative else (good, [good, bad], False)

    env = {}
    made = []

    def make():
        made.append(FakeBuffer(env))
        return made[-1]

    buffer, record = bench.verified_buffer(make, check, 2, env)
    assert len(made) == 2 and made[0].closed and buffer is made[1] and env[bench.FENCE_ENV] == "1"
    assert record["conservative_flags"]["after"] == [["rows 0..4096 differ from their source"]]
    assert record["elements_checked_all_ranks"] == 100 and record["rounds"] == bench.VERIFY_ROUNDS and record["ok"]

    # nothing left to fall back to: the conservative setting is already in force, or there is one rank only
    with pytest.raises(RuntimeError, match="payload check failed"):
        bench.verified_buffer(make, lambda b: check(made[0]), 2, {bench.FENCE_ENV: "1"})
    with pytest.raises(RuntimeError, match="payload check failed"):
        bench.verified_buffer(make, lambda b: check(made[0]), 1, {})

    # the usual case: one buffer, no mention of a fallback
    env2 = {}
    made.clear()
    buffer, record = bench.verified_buffer(make, lambda b: ({"ok": True, "rows_checked": 1, "elements_checked": 7, "problems": []},
                                                            [{"ok": True, "elements_checked": 7, "problems": []}], True), 1, env2)
    assert len(made) == 1 and "conservative_flags" not in record and env2 == {} and record["elements_checked_all_ranks"] == 7


def test_nvlink_audit_reads_counters_and_judges_the_volume():
    import types

    import torch

    from benchmarks import nvlink_audit
    from pcie_ep_b200.ops.reference import route_volume

    class Value:
        def __init__(self, kib, status=0):
            self.nvmlReturn = status
            self.value = types.SimpleNamespace(ullVal=kib)

    class FakeNvml:
        NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX, NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX = 138, 139
        asked = None

        def __init__(self, tx, rx, status=0):
            self.tx, self.rx, self.status = tx, rx, status

        def nvmlDeviceGetFieldValues(self, handle, fields):
            FakeNvml.asked = fields
            return [Value(self.tx, self.status), Value(self.rx)]

    assert nvlink_audit.read_counters(FakeNvml(10, 20), object()) == (10240, 20480)
    assert FakeNvml.asked == [(138, 0xFFFFFFFF), (139, 0xFFFFFFFF)]            # summed over the links, not link 0 alone
    assert nvlink_audit.read_counters(FakeNvml(10, 20, status=3), object()) is None   # a field the driver does not support

    assert nvlink_audit.judge(1000, 1100, 0.9, 1.3)["ok"] and not nvlink_audit.judge(1000, 1600, 0.9, 1.3)["ok"]
    assert not nvlink_audit.judge(1000, 500, 0.9, 1.3)["ok"]
    assert nvlink_audit.judge(0, 4096, 0.9, 1.3)["ok"] and not nvlink_audit.judge(0, 1 << 24, 0.9, 1.3)["ok"]
    assert nvlink_audit.staged_row_bytes(7168, 8, "bf16") == 14336 + 112 and nvlink_audit.staged_row_bytes(7168, 8, "fp8_e4m3") == 7168 + 112

    # two ranks, four experts: token 0 goes to both ranks, token 1 stays on rank 0, token 2 goes to rank 1 twice (one row)
    idx0 = torch.tensor([[0, 2], [1, -1], [2, 3]])
    idx1 = torch.tensor([[0, 1], [3, -1]])
    per_destination = [nvlink_audit.deliveries_per_destination(i, 2, 4) for i in (idx0, idx1)]
    assert per_destination == [[2, 2], [1, 1]]
    volumes = [route_volume(idx0, 0, 2, 4), route_volume(idx1, 1, 2, 4)]
    assert nvlink_audit.expected_traffic(volumes, 0, per_destination, 100, 10) == (2 * 100 * 10, 1 * 100 * 10)
    assert nvlink_audit.expected_traffic(volumes, 1, per_destination, 100, 10) == (1 * 100 * 10, 2 * 100 * 10)


def test_report_shows_what_a_bench_line_says_about_its_payload_checks():
    from benchmarks import report

    assert report.payload_verdict({}) == "-"
    assert report.payload_verdict({"payload_check": {"ok": True}}) == "ok"
    line = {"payload_check": {"ok": True, "conservative_flags": {"mode": "one system-scope fence per row"}},
            "payload_check_after": {"ok": False, "problems": [["rows 0..4096 differ from their source"]]}}
    assert report.payload_verdict(line) == "ok, after: FAILED, one fence per row (fallback)"


def test_benchmark_bandwidth_definitions():
    from benchmarks import benchmark

    volumes = [{"remote_deliveries": 1000}, {"remote_deliveries": 3000}]
    m = benchmark.bandwidth_metrics(volumes, tokens=4096, topk=8, hidden=7168, wire_fp8=False, mean_us=200.0)
    assert m["logical_GBps"] == pytest.approx(4096 * 8 * 7168 * 2 / 200e-6 / 1e9)
    assert m["remote_delivery_GBps_total"] == pytest.approx(4000 * 14336 / 200e-6 / 1e9)
    assert m["remote_delivery_GBps_per_gpu"] == pytest.approx(m["remote_delivery_GBps_total"] / 2)
    fp8 = benchmark.bandwidth_metrics(volumes, 4096, 8, 7168, True, 200.0)
    assert fp8["remote_delivery_GBps_total"] == pytest.approx(4000 * (7168 + 4) / 200e-6 / 1e9)   # codes plus one scale per row
    assert fp8["logical_GBps"] == m["logical_GBps"]                                                # defined on the BF16 input


def test_nccl_log_audit_tells_nvlink_from_shared_memory():
    from benchmarks import nccl_log_audit as audit

    def log(transport, ranks=2, extra=""):
        lines = ["NCCL version 2.28.9+cuda12.9"]
        for r in range(ranks):
            peer = (r + 1) % ranks
            lines.append(f"node7:41{r}:500 [{r}] NCCL INFO ncclCommInitRankConfig comm 0x7f00 rank {r} nranks {ranks} cudaDev {r} nvmlDev {r} "
                         f"busId 1b000 commId 0xdeadbeef - Init COMPLETE")
            lines.append(f"node7:41{r}:501 [{r}] NCCL INFO Channel 00/0 : {r}[{r}] -> {peer}[{peer}] via {transport}")
            lines.append(f"node7:41{r}:501 [{r}] NCCL INFO Channel 01/0 : {r}[{r}] -> {peer}[{peer}] via {transport}")
        return "\n".join(lines) + "\n" + extra

    nvlink = audit.summarise([log("P2P/CUMEM/read", extra="node7:410:502 [0] NCCL INFO Connected NVLS tree\n")])
    assert nvlink["nccl_versions"] == ["2.28.9"] and nvlink["ranks_initialised"] == 2 and nvlink["communicator_sizes"] == [2]
    assert nvlink["connection_lines"] == {"P2P": 4} and nvlink["connected_pairs"] == {"P2P": 2} and nvlink["nvls_active"]
    assert audit.verdict(nvlink, "nvlink", 2) == []
    assert any("via P2P" in p for p in audit.verdict(nvlink, "shm", 2)) and any("NVLS" in p for p in audit.verdict(nvlink, "shm", 2))

    shm = audit.summarise([log("SHM/direct/direct")])
    assert audit.verdict(shm, "shm", 2) == [] and any("via SHM" in p for p in audit.verdict(shm, "nvlink", 2))
    mixed = audit.summarise([log("P2P/IPC"), "node7:9:9 [0] NCCL INFO Channel 00/0 : 0[0] -> 1[1] [send] via NET/Socket/0\n"])
    assert any("via NET" in p for p in audit.verdict(mixed, "nvlink", 2))
    assert any("2 of 8 ranks" in p for p in audit.verdict(nvlink, "nvlink", 8))
    empty = audit.summarise(["nothing of interest\n"])
    assert any("NCCL_DEBUG=INFO" in p for p in audit.verdict(empty, "nvlink", 2))
    # nothing that identifies a machine or a process survives
    assert "node7" not in json.dumps(nvlink) and "deadbeef" not in json.dumps(nvlink)


def test_nccl_log_audit_command_line(tmp_path):
    from benchmarks import nccl_log_audit as audit

    good = tmp_path / "a.log"
    good.write_text("h:1:2 [0] NCCL INFO comm 0x1 rank 0 nranks 1 cudaDev 0 busId 0 commId 0x2 - Init COMPLETE\n"
                    "h:1:2 [0] NCCL INFO Channel 00/0 : 0[0] -> 0[0] via P2P/CUMEM\n")
    assert audit.main(["--expect", "nvlink", "--world", "1", str(good)]) == 0
    assert audit.main(["--expect", "shm", "--world", "1", str(good)]) == 1
    bare = tmp_path / "b.log"
    bare.write_text("no NCCL lines\n")
    assert audit.main(["--expect", "nvlink", "--world", "1", str(bare)]) == 2


def test_bench_clock_sampler_takes_direct_samples_and_reports_them():
    import bench

    class FakeNvml:
        NVML_CLOCK_SM = 1
        calls = 0

        def nvmlDeviceGetClockInfo(self, handle, kind):
            FakeNvml.calls += 1
            return 1965 if FakeNvml.calls != 2 else 1410

        def nvmlDeviceGetCurrentClocksEventReasons(self, handle):
            return 0x4 if FakeNvml.calls == 2 else 0          # the second sample saw the power cap

    sampler = bench.ClockSampler(0)
    sampler._nvml, sampler._handle, sampler.max_clock = FakeNvml(), object(), 1965.0
    for _ in range(3):
        sampler.sample_now()
    record = sampler.stop()                                    # (the thread was never started)
    assert record["samples"] == 3 and record["samples_after_last_launch"] == 3
    assert record["sm_mhz"] == 1965.0 and record["sm_max_mhz"] == 1965.0 and record["reasons"] == ["sw_power_cap"]
    sampler._nvml = type("Broken", (), {"NVML_CLOCK_SM": 1, "nvmlDeviceGetClockInfo": lambda *a: 1 / 0})()
    sampler.sample_now()                                       # a failing query is skipped, never raised
    assert len(sampler.samples) == 3
