"""Digests that let many ranks prove a bit-exact dispatch without shipping the rows around.

``dispatch_digest`` folds what ``PyTorchAllToAll.dispatch`` returns (reference.py:148) --
per-expert counts, the valid prefix of every expert's rows and its ``(expert, source rank,
token, k)`` records, in the reference's order -- into three 64-bit integers with
position-dependent multipliers, so a missing, repeated, misplaced or altered row changes
them.  A rank computes the digest of what its GPU holds, rank 0 computes the digest of the
expectation, and only the integers travel.
"""
from __future__ import annotations

from typing import Tuple

import torch


def _fold(values: torch.Tensor) -> int:
    """Sum of (value + 1) * multiplier(position) in wrapping int64 arithmetic."""
    v = values.reshape(-1).to(torch.int64)
    if v.numel() == 0:
        return 0
    pos = torch.arange(v.numel(), dtype=torch.int64, device=v.device)
    mult = (pos * 2654435761 + 40503) % 1000003 + 1
    return int(((v + 1) * mult).sum().item())


def dispatch_digest(counts: torch.Tensor, rows: torch.Tensor, meta: torch.Tensor) -> Tuple[int, int, int]:
    """``counts`` [L] int32; ``rows`` / ``meta`` the valid prefixes of all experts concatenated
    (``[sum(counts), H]`` of a 16-bit type, ``[sum(counts), 5]`` int32)."""
    return (_fold(counts.to(torch.int64)),
            _fold(rows.contiguous().view(torch.int16)),
            _fold(meta))


def compact_dispatch(counts: torch.Tensor, rows: torch.Tensor, meta: torch.Tensor):
    """Padded ``[L, max_recv, ...]`` buffers -> concatenated valid prefixes."""
    n = counts.tolist()
    if sum(n) == 0:
        return rows[:0, 0] if rows.dim() == 3 else rows[:0], meta[:0, 0] if meta.dim() == 3 else meta[:0]
    r = torch.cat([rows[e, : n[e]] for e in range(len(n))], 0)
    m = torch.cat([meta[e, : n[e]] for e in range(len(n))], 0)
    return r, m
