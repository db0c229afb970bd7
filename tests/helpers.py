"""Shared input generators and the slow, per-token statement of the semantics used to check the
vectorised oracle (modelled on how the reference's tests build their inputs,
tests/test_correctness.py:31-92, but written independently)."""

from __future__ import annotations

import socket
from typing import List, Optional, Tuple

import torch


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_inputs(rank: int, world: int, tokens: int, hidden: int, experts: int, topk: int, pattern: str = "random",
                seed: int = 7, dtype: torch.dtype = torch.bfloat16, weights: bool = True):
    g = torch.Generator().manual_seed(seed + rank * 7919)
    local = experts // world
    if pattern == "local":
        idx = (torch.arange(topk) % local + rank * local).repeat(tokens, 1)
    elif pattern == "multicast":
        ids = [dest * local + le for le in range(local) for dest in range(world)]
        idx = torch.tensor(ids[:topk], dtype=torch.int64).repeat(tokens, 1)
    elif pattern == "hotspot":
        idx = torch.arange(topk).repeat(tokens, 1)
    else:
        idx = torch.rand(tokens, experts, generator=g).topk(topk, dim=1).indices
    idx = idx.to(torch.int64)
    if pattern == "none":
        idx.fill_(-1)
    elif pattern == "partial" and tokens:
        idx[:, ::3] = -1
    w = torch.rand(tokens, topk, generator=g).to(torch.float32)
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    # make token identity visible in the payload as well
    if tokens and hidden >= 2:
        x[:, 0] = (torch.arange(tokens) % 251).to(dtype)
        x[:, 1] = float(rank)
    return x.contiguous(), idx.contiguous(), (w.contiguous() if weights else None)


def enumerate_reference(inputs, rank: int, experts: int, alignment: int):
    """Token-by-token enumeration: unique rows, per-expert rows, counts, offsets, U and F."""
    world = len(inputs)
    local = experts // world
    topk = inputs[0][1].shape[1]
    unique, expanded = [], [[] for _ in range(local)]
    writes = reads = deliveries = 0
    for source, (x, idx, w) in enumerate(inputs):
        for token in range(x.shape[0]):
            route = idx[token].tolist()
            dests = {e // local for e in route if e >= 0}
            if source == rank:
                if any(d != rank for d in dests):
                    writes += 1
                deliveries += len(dests - {rank})
            slots = [s for s in range(topk) if route[s] >= 0 and route[s] // local == rank]
            if not slots:
                continue
            if source != rank:
                reads += 1
            out_idx = [-1] * topk
            out_w = [0.0] * topk
            for s in slots:
                le = route[s] % local
                out_idx[s] = le
                out_w[s] = float(w[token, s]) if w is not None else 1.0
                expanded[le].append((source, token, s, out_w[s]))
            unique.append((source, token, out_idx, out_w))
    counts = [len(rows) for rows in expanded]
    offsets = [0]
    for count in counts:
        offsets.append(offsets[-1] + (count + alignment - 1) // alignment * alignment)
    return unique, expanded, counts, offsets, writes, reads, deliveries
