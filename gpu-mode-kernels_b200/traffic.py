"""Algorithmic traffic of one dispatch+combine, fixed by the routing alone.

For rank r: ``egress[r]`` = (token,k) pairs on r whose expert lives on another
rank, ``ingress[r]`` = pairs of other ranks routed to r.  Dispatch moves
``egress*row_d`` bytes out and ``ingress*row_d`` in; combine the reverse with
``row_c``.  NVLink is full duplex, so the time floor of a phase on rank r is
``max(egress, ingress) * row / link_bandwidth`` and the job's floor is the
maximum over ranks.  The ``dedup`` figures count one row per (token,
destination rank) instead of one per pair (what the DEDUP/FP8 payloads put on
the wire in dispatch).
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

NVLINK_NOMINAL_GBS = 900.0   # per direction per GPU, NVLink 5: the peak every NVLink fraction is quoted against


def pair_counts(indices: Sequence[torch.Tensor], num_experts: int, world_size: int):
    """[src, dst] matrices: pairs, and distinct (token, dst) rows."""
    L = num_experts // world_size
    pairs = torch.zeros(world_size, world_size, dtype=torch.int64)
    rows = torch.zeros(world_size, world_size, dtype=torch.int64)
    for s, idx in enumerate(indices):
        dst = idx.to(torch.int64).cpu() // L
        for d in range(world_size):
            hit = dst == d
            pairs[s, d] = int(hit.sum())
            rows[s, d] = int(hit.any(dim=1).sum()) if hit.numel() else 0
    return pairs, rows


def row_bytes(hidden_dim: int, payload: str = "direct") -> int:
    if payload == "fp8":
        return hidden_dim + 4 * (hidden_dim // 128)
    return 2 * hidden_dim


def summarize(indices: Sequence[torch.Tensor], num_experts: int, world_size: int, hidden_dim: int,
              payload: str = "direct", combine: str = "pull") -> Dict[str, float]:
    """``algorithmic_bytes`` counts one row per (token, k) pair in both directions whatever the
    implementation does; ``wire_bytes`` is what the chosen payload / combine mode really moves
    (``combine="push"`` returns one partial row per (token, expert rank) instead of one per pair)."""
    pairs, rows = pair_counts(indices, num_experts, world_size)
    off = ~torch.eye(world_size, dtype=torch.bool)
    eg = (pairs * off).sum(1)
    ig = (pairs * off).sum(0)
    eg_d = (rows * off).sum(1)
    ig_d = (rows * off).sum(0)
    busiest = int(torch.maximum(eg, ig).max()) if world_size > 1 else 0
    busiest_d = int(torch.maximum(eg_d, ig_d).max()) if world_size > 1 else 0
    row_d, row_c = row_bytes(hidden_dim, payload), 2 * hidden_dim
    alg = busiest * (row_d + row_c)  # bytes per direction on the busiest rank, dispatch + combine
    wire_dispatch_rows = busiest_d if payload in ("dedup", "fp8") else busiest
    wire = wire_dispatch_rows * row_d + (busiest_d if combine == "push" else busiest) * row_c
    total_pairs = int(pairs.sum())
    return dict(
        busiest_rows=busiest, busiest_rows_dedup=busiest_d,
        algorithmic_bytes=alg, wire_bytes=wire,
        t_roof_us_nominal=alg / (NVLINK_NOMINAL_GBS * 1e3) if world_size > 1 else 0.0,
        t_wire_us_nominal=wire / (NVLINK_NOMINAL_GBS * 1e3) if world_size > 1 else 0.0,
        total_pairs=total_pairs, local_pairs=int(pairs.diagonal().sum()),
    )


def hbm_bytes_single_rank(num_tokens: int, top_k: int, hidden_dim: int) -> Dict[str, int]:
    """Algorithmic HBM bytes per kernel when every expert is local (world size 1)."""
    row = 2 * hidden_dim
    pairs = num_tokens * top_k
    return dict(
        route=pairs * 8,
        dispatch_send=(num_tokens + pairs) * row,  # read each token row once, write one row per pair
        recv_expert=2 * pairs * row,               # read and rewrite every received row
        combine=(pairs + num_tokens) * row,        # read one row per pair, write one per token
    )
