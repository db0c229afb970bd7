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
