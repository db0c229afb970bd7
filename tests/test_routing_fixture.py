"""Routing fixtures: determinism, routing contract, skew statistics, tamper rejection
(reference: tests/test_routing_fixture.py)."""

import json

import numpy as np
import pytest
import torch

from benchmarks.routing_fixture import FixtureSpec, expert_popularity, load_fixture, make_routes, route_statistics, save_fixture


@pytest.mark.parametrize("profile", ["uniform", "hotspot_20_80", "zipf"])
def test_routes_are_deterministic_and_valid(profile):
    spec = FixtureSpec(profile, 256, 64, 4, 4)
    for rank in range(4):
        idx, w = make_routes(spec, rank)
        idx2, w2 = make_routes(spec, rank)
        assert torch.equal(idx, idx2) and torch.equal(w, w2)
        assert idx.shape == (256, 4) and idx.dtype == torch.int64 and w.dtype == torch.float32
        assert idx.min() >= 0 and idx.max() < 64
        ordered = idx.sort(dim=1).values
        assert not (ordered[:, 1:] == ordered[:, :-1]).any()
        assert torch.allclose(w.sum(dim=1), torch.ones(256), atol=1e-5)
    assert not torch.equal(make_routes(spec, 0)[0], make_routes(spec, 1)[0])


def test_skew_profiles_are_skewed():
    uniform = route_statistics(FixtureSpec("uniform", 2048, 256, 4, 8))
    hotspot = route_statistics(FixtureSpec("hotspot_20_80", 2048, 256, 4, 8))
    zipf = route_statistics(FixtureSpec("zipf", 2048, 256, 4, 8))
    assert uniform["expert_cv"] < 0.2
    assert hotspot["expert_cv"] > 0.8 and zipf["expert_cv"] > 0.8
    mass = expert_popularity(FixtureSpec("hotspot_20_80", 1, 256, 4, 8))
    top = mass.sort(descending=True).values[:51].sum()
    assert abs(float(top) - 0.8) < 1e-6
    assert hotspot["remote_share_of_allgather"] < uniform["remote_share_of_allgather"] + 0.2


def test_save_load_and_tamper_rejection(tmp_path):
    spec = FixtureSpec("zipf", 64, 32, 4, 2)
    save_fixture(spec, tmp_path)
    manifest = tmp_path / f"{spec.name()}.json"
    loaded, routes = load_fixture(manifest)
    assert loaded == spec and torch.equal(routes[1][0], make_routes(spec, 1)[0])
    data = dict(np.load(manifest.with_suffix(".npz")))
    data["idx_0"][0, 0] = (data["idx_0"][0, 0] + 1) % 32
    np.savez(manifest.with_suffix(".npz"), **data)
    with pytest.raises(ValueError, match="SHA-256"):
        load_fixture(manifest)
    info = json.loads(manifest.read_text())
    info["spec"]["world"] = 3
    manifest.write_text(json.dumps(info))
    with pytest.raises(ValueError):
        load_fixture(manifest)


def test_calibrated_profile_matches_the_published_moments():
    from benchmarks.routing_fixture import CALIBRATED_CV, CALIBRATED_MAX_OVER_MEAN, calibrated_spectrum

    spectrum = calibrated_spectrum(256, 4)
    loads = spectrum * 256 / 4
    assert abs(float(spectrum.sum()) - 4.0) < 1e-9 and float(spectrum.max()) <= 1.0
    assert abs(float(loads.std(unbiased=False) / loads.mean()) - CALIBRATED_CV) < 1e-6
    assert abs(float(loads.max() / loads.mean()) - CALIBRATED_MAX_OVER_MEAN) < 1e-9
    stats = route_statistics(FixtureSpec("nvidia_calibrated", 4096, 256, 4, 8))
    assert abs(stats["expert_cv"] - CALIBRATED_CV) < 0.05 and abs(stats["expert_max_over_mean"] - CALIBRATED_MAX_OVER_MEAN) < 0.6
    idx, _ = make_routes(FixtureSpec("nvidia_calibrated", 512, 256, 4, 8), 3)
    ordered = idx.sort(dim=1).values
    assert not (ordered[:, 1:] == ordered[:, :-1]).any() and idx.min() >= 0 and idx.max() < 256
    with pytest.raises(ValueError):
        calibrated_spectrum(16, 4)  # the heaviest expert would need an inclusion probability above one


def test_committed_frozen_fixtures_load_and_match_their_generators():
    from benchmarks.routing_fixture import FROZEN_SPECS, frozen_manifest

    for spec in FROZEN_SPECS:
        loaded, routes = load_fixture(frozen_manifest(spec.profile), tokens=128)
        assert loaded == spec and len(routes) == 8 and routes[0][0].shape == (128, 4)
        assert torch.equal(routes[5][0], make_routes(spec, 5)[0][:128])  # frozen file == its generator
    with pytest.raises(ValueError):
        load_fixture(frozen_manifest("zipf"), tokens=9000)
