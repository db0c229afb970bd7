"""Frozen routing fixtures: reproducible expert ids and weights for skewed-load benchmarks.

Profiles
    ``uniform``        distinct uniform expert ids per token (``rand().topk``), as the headline benchmark.
    ``hotspot_20_80``  20 % of the experts receive 80 % of the routing mass; ids drawn without
                       replacement with the Gumbel top-k trick.
    ``zipf``           expert popularity proportional to ``1 / rank**s`` (default s = 1.1) over a fixed
                       random permutation of the experts; Gumbel top-k as above.
    ``nvidia_calibrated``  per-expert *inclusion probabilities* whose coefficient of variation (164.1 / 128) and
                       maximum over mean (11.948) equal the expert-load figures NVIDIA published for DeepSeek-R1
                       without load balancing (TensorRT-LLM "Scaling Expert Parallelism", table 1): one expert at
                       the maximum, the others on a power-law tail whose exponent is solved for; tokens are drawn
                       by systematic sampling over a random permutation, which picks exactly ``topk`` distinct
                       experts with exactly those inclusion probabilities.  A synthetic moment match, not a trace.

Parity: the reference's ``benchmarks/routing_fixture.py`` (generators, NPZ + JSON manifest with hashes, strict
loader) and its committed ``benchmarks/data/top4_skew`` files.  A fixture is a pure function of
``(profile, tokens, experts, topk, world, seed)``, is written to ``<name>.npz`` + ``<name>.json`` and is
verified against its manifest (shape, dtype, SHA-256, distinct ids per token, range) when loaded.  The files
under ``benchmarks/data/top4_skew`` are frozen at 8192 tokens per rank; a benchmark at fewer tokens takes the
first T rows of every rank's table, so all sizes see the same routes in every run.

    python -m benchmarks.routing_fixture --write benchmarks/data/top4_skew     # regenerate the committed files
    python -m benchmarks.routing_fixture --check benchmarks/data/top4_skew     # verify them against their manifests
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

PROFILES = ("uniform", "hotspot_20_80", "zipf", "nvidia_calibrated")
CALIBRATED_CV = 164.1 / 128.0
CALIBRATED_MAX_OVER_MEAN = 11.948
DEFAULT_SEED = 20261024


@dataclass(frozen=True)
class FixtureSpec:
    profile: str
    tokens: int
    experts: int
    topk: int
    world: int
    seed: int = DEFAULT_SEED
    zipf_s: float = 1.1

    def name(self) -> str:
        return f"{self.profile}_t{self.tokens}_e{self.experts}_k{self.topk}_w{self.world}_s{self.seed}"


def expert_popularity(spec: FixtureSpec) -> torch.Tensor:
    """Probability mass of every expert (sums to 1); identical on every rank."""
    g = torch.Generator().manual_seed(spec.seed)
    if spec.profile == "uniform":
        return torch.full((spec.experts,), 1.0 / spec.experts, dtype=torch.float64)
    order = torch.randperm(spec.experts, generator=g)
    mass = torch.empty(spec.experts, dtype=torch.float64)
    if spec.profile == "hotspot_20_80":
        hot = max(1, round(0.2 * spec.experts))
        mass[order[:hot]] = 0.8 / hot
        mass[order[hot:]] = 0.2 / max(1, spec.experts - hot)
    elif spec.profile == "zipf":
        ranks = torch.arange(1, spec.experts + 1, dtype=torch.float64)
        weights = ranks.pow(-spec.zipf_s)
        mass[order] = weights / weights.sum()
    elif spec.profile == "nvidia_calibrated":
        mass[order] = calibrated_spectrum(spec.experts, spec.topk) / spec.topk
    else:
        raise ValueError(f"unknown profile {spec.profile!r}; choose from {PROFILES}")
    return mass / mass.sum()


def calibrated_spectrum(experts: int, topk: int) -> torch.Tensor:
    """Inclusion probabilities (descending, summing to ``topk``) with the published load moments.

    Relative loads r_e have mean 1: r_0 is pinned to the published maximum over mean, the other E - 1 follow
    ``rank ** -a`` scaled to the remaining mass; ``a`` is found by bisection so that the coefficient of variation
    of all E loads hits the published value (the sum of squares grows monotonically with ``a``)."""
    top = CALIBRATED_MAX_OVER_MEAN
    if top * topk / experts > 1.0:
        raise ValueError("too few experts for this top-k: the heaviest expert's inclusion probability would exceed one")
    want_square_sum = experts * (1.0 + CALIBRATED_CV ** 2) - top ** 2
    ranks = torch.arange(1, experts, dtype=torch.float64)

    def tail_for(a: float) -> torch.Tensor:
        t = ranks.pow(-a)
        return t * ((experts - top) / t.sum())

    lo, hi = 0.0, 4.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if float(tail_for(mid).square().sum()) < want_square_sum:
            lo = mid
        else:
            hi = mid
    tail = tail_for(0.5 * (lo + hi))
    if float(tail.max()) > top:
        raise ValueError("the tail overtakes the pinned maximum: moments not reachable for this expert count")
    return torch.cat([torch.tensor([top], dtype=torch.float64), tail]) * (topk / experts)


def _systematic_sample(inclusion: torch.Tensor, tokens: int, topk: int, g: torch.Generator) -> torch.Tensor:
    """Exactly ``topk`` distinct experts per token, expert e with probability ``inclusion[e]`` (sum = topk, each <= 1):
    lay the probabilities end to end in a random order per token and pick the experts under the points
    u, u + 1, ..., u + topk - 1 for one uniform u."""
    experts = inclusion.numel()
    out = torch.empty(tokens, topk, dtype=torch.int64)
    for lo in range(0, tokens, 2048):
        n = min(2048, tokens - lo)
        order = torch.rand(n, experts, generator=g).argsort(dim=1)
        edges = inclusion[order].cumsum(dim=1)
        edges[:, -1] = float(topk)  # guard the last edge against rounding
        points = torch.rand(n, 1, generator=g, dtype=torch.float64) + torch.arange(topk, dtype=torch.float64)
        picked = torch.searchsorted(edges, points, right=True).clamp_(max=experts - 1)
        chosen = order.gather(1, picked)
        shuffle = torch.rand(n, topk, generator=g).argsort(dim=1)  # no meaning in the slot order
        out[lo:lo + n] = chosen.gather(1, shuffle)
    return out


def make_routes(spec: FixtureSpec, rank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(topk_idx int64 [T, K], topk_weights float32 [T, K])`` of one rank; ids distinct within a token."""
    if not 0 <= rank < spec.world:
        raise ValueError("rank out of range")
    if spec.topk > spec.experts:
        raise ValueError("topk exceeds the number of experts")
    g = torch.Generator().manual_seed(spec.seed + rank * 104729 + spec.tokens)
    if spec.profile == "uniform":
        idx = torch.rand(spec.tokens, spec.experts, generator=g).topk(spec.topk, dim=1).indices
    elif spec.profile == "nvidia_calibrated":
        idx = _systematic_sample(expert_popularity(spec) * spec.topk, spec.tokens, spec.topk, g)
    else:
        # Gumbel top-k: sampling without replacement proportional to the popularity
        log_mass = expert_popularity(spec).log().float()
        uniform = torch.rand(spec.tokens, spec.experts, generator=g).clamp_(1e-12, 1.0 - 1e-7)
        gumbel = -torch.log(-torch.log(uniform))
        idx = (log_mass.unsqueeze(0) + gumbel).topk(spec.topk, dim=1).indices
    weights = torch.softmax(torch.randn(spec.tokens, spec.topk, generator=g), dim=1).to(torch.float32)
    return idx.to(torch.int64).contiguous(), weights.contiguous()


def route_statistics(spec: FixtureSpec) -> Dict[str, float]:
    """Load statistics over all ranks: expert CV, max/mean, share of an all-gather that really moves."""
    counts = torch.zeros(spec.experts, dtype=torch.float64)
    local = spec.experts // spec.world
    remote_deliveries = 0
    for rank in range(spec.world):
        idx, _ = make_routes(spec, rank)
        counts += torch.bincount(idx.flatten(), minlength=spec.experts).double()
        owners = idx // local
        hit = torch.zeros(spec.tokens, spec.world, dtype=torch.bool)
        hit.scatter_(1, owners, True)
        hit[:, rank] = False
        remote_deliveries += int(hit.sum())
    mean = counts.mean().item()
    return {
        "expert_cv": float(counts.std(unbiased=False).item() / mean) if mean else 0.0,
        "expert_max_over_mean": float(counts.max().item() / mean) if mean else 0.0,
        "remote_deliveries": remote_deliveries,
        "remote_share_of_allgather": remote_deliveries / float(spec.world * spec.tokens * max(1, spec.world - 1)),
    }


def _sha256(array: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def save_fixture(spec: FixtureSpec, directory: Path) -> Path:
    """Write ``<name>.npz`` (per-rank ids and weights) and ``<name>.json`` (manifest with hashes)."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    arrays: Dict[str, np.ndarray] = {}
    hashes: Dict[str, str] = {}
    for rank in range(spec.world):
        idx, weights = make_routes(spec, rank)
        arrays[f"idx_{rank}"] = idx.numpy()
        arrays[f"weights_{rank}"] = weights.numpy()
    for key, value in arrays.items():
        hashes[key] = _sha256(value)
    np.savez_compressed(directory / f"{spec.name()}.npz", **arrays)
    manifest = {"spec": asdict(spec), "sha256": hashes, "statistics": route_statistics(spec)}
    (directory / f"{spec.name()}.json").write_text(json.dumps(manifest, indent=2, sort_keys=True))
    return directory / f"{spec.name()}.npz"


def load_fixture(manifest_path: Path, tokens: int = 0) -> Tuple[FixtureSpec, List[Tuple[torch.Tensor, torch.Tensor]]]:
    """Strict loader: refuses files that do not match their manifest or violate the routing contract.

    ``tokens`` > 0 returns the first ``tokens`` rows of every rank's table (after the whole file has been verified)."""
    manifest_path = Path(manifest_path)
    manifest = json.loads(manifest_path.read_text())
    spec = FixtureSpec(**manifest["spec"])
    data = np.load(manifest_path.with_suffix(".npz"))
    expected_keys = {f"{kind}_{rank}" for kind in ("idx", "weights") for rank in range(spec.world)}
    if set(data.files) != expected_keys:
        raise ValueError("fixture arrays do not match the manifest's world size")
    routes = []
    for rank in range(spec.world):
        idx, weights = data[f"idx_{rank}"], data[f"weights_{rank}"]
        if idx.shape != (spec.tokens, spec.topk) or idx.dtype != np.int64:
            raise ValueError(f"rank {rank}: expert ids have the wrong shape or dtype")
        if weights.shape != (spec.tokens, spec.topk) or weights.dtype != np.float32:
            raise ValueError(f"rank {rank}: weights have the wrong shape or dtype")
        for key, array in ((f"idx_{rank}", idx), (f"weights_{rank}", weights)):
            if _sha256(array) != manifest["sha256"].get(key):
                raise ValueError(f"{key}: SHA-256 differs from the manifest (file was modified)")
        if idx.min(initial=0) < 0 or idx.max(initial=0) >= spec.experts:
            raise ValueError(f"rank {rank}: expert id out of range")
        ordered = np.sort(idx, axis=1)
        if spec.topk > 1 and (ordered[:, 1:] == ordered[:, :-1]).any():
            raise ValueError(f"rank {rank}: a token repeats an expert")
        routes.append((torch.from_numpy(idx.copy()), torch.from_numpy(weights.copy())))
    if tokens:
        if tokens > spec.tokens:
            raise ValueError(f"the fixture holds {spec.tokens} tokens per rank, {tokens} were asked for")
        routes = [(idx[:tokens].contiguous(), weights[:tokens].contiguous()) for idx, weights in routes]
    return spec, routes


FROZEN_DIRECTORY = Path(__file__).resolve().parent / "data" / "top4_skew"
FROZEN_SPECS = tuple(FixtureSpec(profile, 8192, 256, 4, 8) for profile in ("hotspot_20_80", "zipf", "nvidia_calibrated"))


def frozen_manifest(profile: str) -> Path:
    for spec in FROZEN_SPECS:
        if spec.profile == profile:
            return FROZEN_DIRECTORY / f"{spec.name()}.json"
    raise ValueError(f"no frozen fixture for profile {profile!r}")


def main() -> None:
    import argparse

    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--write", type=Path, help="directory to (re)generate the frozen fixtures in")
    parser.add_argument("--check", type=Path, help="directory whose fixtures are verified against their manifests")
    args = parser.parse_args()
    if args.write:
        for spec in FROZEN_SPECS:
            print(save_fixture(spec, args.write))
    if args.check:
        for manifest in sorted(Path(args.check).glob("*.json")):
            spec, routes = load_fixture(manifest)
            print(f"{manifest.name}: ok ({spec.world} ranks x {spec.tokens} tokens, statistics {route_statistics(spec)})")


if __name__ == "__main__":
    main()
