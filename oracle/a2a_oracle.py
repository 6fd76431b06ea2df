"""CPU restatement of the reference MoE all-to-all path.  TEST INFRASTRUCTURE ONLY.

This file is the checker: tests, the smoke check and the CPU-baseline legs of
the benchmark may call it; the shipped GPU path never does.

It restates, in CPU PyTorch, the algorithm of the reference's pure-Python
implementation (file ``amd-distributed/all2all/reference.py`` of
gau-nernst/gpu-mode-kernels).  Two forms are kept, both pinned on golden
vectors produced by running the reference itself under gloo
(``tests/golden/make_golden.py`` made them; ``tests/test_oracle_golden.py``
checks them):

* ``PortAllToAll`` / ``port_ref_kernel`` -- the literal per-rank port: one
  process per rank, ``torch.distributed.all_to_all_single`` for the six
  exchanges, the same Python loops in the same order.  This is what the
  CPU-baseline timing runs.
* ``simulate`` -- all ranks in one process, vectorised: the exchange is a list
  shuffle, regrouping is a stable sort.  This is what parity checks use at
  full problem sizes.

Semantics both forms reproduce (reference.py line numbers):

* sender order: pairs enumerated ``for t: for k`` (:79-80); per destination
  rank ``dst = e // L`` (:81) the rows keep that order (:83,93); meta row is
  ``[global_expert, src_rank, t, k, 0]`` (:84-86).
* receiver order: arrival is source rank ascending (:107-112); regroup appends
  to local expert ``e % L`` in arrival order (:140-146).  Hence rows of one
  expert are ordered by ``(src_rank, t, k)`` and ``expert_num_tokens[e]`` is
  the number of pairs routed to ``e``.
* expert placeholder: ``expert_x.to(out_dtype) * (1 + rank)`` (:262) -- fp32
  multiply, one round-to-nearest-even into ``out_dtype``.
* combine: rows return grouped by expert rank ascending, within a rank by
  ``(local_expert, slot)`` (:170-179,210-215); ``out[t] += float(row) * w[t,k]``
  in that order with a rounding to ``out_dtype`` after every add (:226-232);
  ``out`` starts as zeros ``[max_num_tokens, H]`` and ``[:num_tokens]`` is
  returned (:263-272).
"""
from __future__ import annotations

import dataclasses
from typing import List, Sequence

import torch

META_DIM = 5  # global_exp, src_rank, src_token, src_k, pad  (reference.py:56)


# --------------------------------------------------------------------------
# literal per-rank port (one process per rank, torch.distributed exchange)
# --------------------------------------------------------------------------
class PortAllToAll:
    """Per-rank port of ``PyTorchAllToAll`` (reference.py:55-234)."""

    def __init__(self, cfg, rank: int, world_size: int, dist=None):
        if dist is None:
            import torch.distributed as dist  # noqa: PLW0621
        self.dist = dist
        self.cfg = cfg
        self.rank = rank
        self.world_size = world_size
        self.num_local_experts = cfg.num_experts // world_size  # :63
        self.max_recv = cfg.max_num_tokens * world_size  # :65

    def dispatch(self, dp_x: torch.Tensor, indices: torch.Tensor):
        """reference.py:68-148."""
        cfg, ws, L = self.cfg, self.world_size, self.num_local_experts
        dev = dp_x.device
        send_counts = [0] * ws
        token_map: List[List[int]] = [[] for _ in range(ws)]
        meta_map: List[List[int]] = [[] for _ in range(ws)]
        for t, experts in enumerate(indices.tolist()):  # :79-86
            for k, e in enumerate(experts):
                d = e // L
                send_counts[d] += 1
                token_map[d].append(t)
                meta_map[d].extend([e, self.rank, t, k, 0])
        send_counts_t = torch.tensor(send_counts, dtype=torch.long, device=dev)
        recv_counts_t = torch.empty(ws, dtype=torch.long, device=dev)
        self.dist.all_to_all_single(recv_counts_t, send_counts_t)  # :91
        send_buf = torch.cat([dp_x[ids] for ids in token_map], dim=0)  # :93
        total_recv = int(recv_counts_t.sum().item())
        recv_buf = torch.empty(total_recv, cfg.hidden_dim, dtype=cfg.in_dtype, device=dev)
        send_meta = torch.tensor([v for sub in meta_map for v in sub], dtype=torch.int32,
                                 device=dev).view(-1, META_DIM)
        recv_meta = torch.empty(total_recv, META_DIM, dtype=torch.int32, device=dev)
        rc, sc = recv_counts_t.tolist(), send_counts_t.tolist()
        self.dist.all_to_all_single(recv_buf, send_buf, output_split_sizes=rc, input_split_sizes=sc)  # :107
        self.dist.all_to_all_single(  # :114
            recv_meta.view(-1), send_meta.view(-1),
            output_split_sizes=[c * META_DIM for c in rc],
            input_split_sizes=[c * META_DIM for c in sc],
        )
        recv_meta = recv_meta.view(-1, META_DIM)
        expert_num_tokens = torch.zeros(L, dtype=torch.int32, device=dev)
        expert_x = torch.empty((L, self.max_recv, cfg.hidden_dim), dtype=cfg.in_dtype, device=dev)
        expert_meta = torch.empty((L, self.max_recv, META_DIM), dtype=torch.int32, device=dev)
        for i in range(total_recv):  # :140-146
            local = int(recv_meta[i, 0].item()) % L
            expert_x[local, expert_num_tokens[local]] = recv_buf[i]
            expert_meta[local, expert_num_tokens[local]] = recv_meta[i]
            expert_num_tokens[local] += 1
        return expert_num_tokens, expert_x, expert_meta

    def combine(self, out_tokens, weights, expert_meta, expert_y, expert_num_tokens):
        """reference.py:151-234."""
        cfg, ws = self.cfg, self.world_size
        dev = out_tokens.device
        send_counts = [0] * ws
        y_map: List[list] = [[] for _ in range(ws)]
        meta_map: List[List[int]] = [[] for _ in range(ws)]
        for local in range(self.num_local_experts):  # :170-179
            cnt = int(expert_num_tokens[local].item())
            for j in range(cnt):
                meta = expert_meta[local, j]
                d = int(meta[1].item())
                send_counts[d] += 1
                y_map[d].append(expert_y[local, j].unsqueeze(0))
                meta_map[d].extend(meta.tolist())
        send_counts_t = torch.tensor(send_counts, dtype=torch.long, device=dev)
        recv_counts_t = torch.empty(ws, dtype=torch.long, device=dev)
        self.dist.all_to_all_single(recv_counts_t, send_counts_t)  # :185
        parts = [torch.cat(s, dim=0) if s else torch.empty((0, cfg.hidden_dim), dtype=cfg.out_dtype, device=dev)
                 for s in y_map]
        send_buf = torch.cat(parts, dim=0)
        send_meta = torch.tensor([v for sub in meta_map for v in sub], dtype=torch.int32,
                                 device=dev).view(-1, META_DIM)
        total_recv = int(recv_counts_t.sum().item())
        recv_buf = torch.empty(total_recv, cfg.hidden_dim, dtype=cfg.out_dtype, device=dev)
        recv_meta = torch.empty(total_recv, META_DIM, dtype=torch.int32, device=dev)
        rc, sc = recv_counts_t.tolist(), send_counts_t.tolist()
        self.dist.all_to_all_single(recv_buf, send_buf, output_split_sizes=rc, input_split_sizes=sc)  # :210
        self.dist.all_to_all_single(  # :217
            recv_meta.view(-1), send_meta.view(-1),
            output_split_sizes=[c * META_DIM for c in rc],
            input_split_sizes=[c * META_DIM for c in sc],
        )
        recv_meta = recv_meta.view(-1, META_DIM)
        for i in range(total_recv):  # :227-232
            t = int(recv_meta[i, 2].item())
            k = int(recv_meta[i, 3].item())
            w = weights[t, k].to(torch.float32)
            out_tokens[t] += recv_buf[i].to(torch.float32) * w
        return out_tokens


def port_expert_op(expert_x: torch.Tensor, out_dtype, rank: int, expert_num_tokens=None) -> torch.Tensor:
    """The placeholder expert op (reference.py:262).

    With ``expert_num_tokens`` given only the valid prefix of every expert is
    computed (the rest of the padded buffer is uninitialised and never read
    downstream); without it the whole padded buffer is multiplied as the
    reference does.
    """
    if expert_num_tokens is None:
        return expert_x.to(out_dtype) * (1 + rank)
    out = torch.empty_like(expert_x, dtype=out_dtype)
    for e, n in enumerate(expert_num_tokens.tolist()):
        out[e, :n] = expert_x[e, :n].to(out_dtype) * (1 + rank)
    return out


def port_ref_kernel(data, dist=None, valid_rows_only: bool = False) -> torch.Tensor:
    """Per-rank port of ``ref_kernel`` (reference.py:256-272)."""
    cfg, rank_data, rank, world_size = data
    ata = PortAllToAll(cfg, rank, world_size, dist=dist)
    expert_num, expert_x, expert_meta = ata.dispatch(rank_data.x, rank_data.indices)
    expert_y = port_expert_op(expert_x, cfg.out_dtype, rank, expert_num if valid_rows_only else None)
    y = torch.zeros(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=rank_data.x.device)
    ata.combine(y, rank_data.weights, expert_meta, expert_y, expert_num)
    return y[: rank_data.num_tokens]


# --------------------------------------------------------------------------
# all ranks in one process, vectorised
# --------------------------------------------------------------------------
@dataclasses.dataclass
class RankDispatch:
    """What ``dispatch`` returns on one rank, without the uninitialised padding.

    ``rows``/``meta`` hold the valid prefix of every local expert, concatenated
    in local-expert order; expert ``e`` owns ``rows[offsets[e]:offsets[e+1]]``.
    """

    expert_num_tokens: torch.Tensor  # [L] int32
    rows: torch.Tensor  # [sum(n_e), H] in_dtype
    meta: torch.Tensor  # [sum(n_e), 5] int32
    offsets: torch.Tensor  # [L+1] int64

    def padded(self, max_recv: int):
        """The reference's ``[L, max_recv, ...]`` layout with zeros where it has garbage."""
        L = self.expert_num_tokens.numel()
        x = torch.zeros(L, max_recv, self.rows.shape[1], dtype=self.rows.dtype)
        m = torch.zeros(L, max_recv, META_DIM, dtype=torch.int32)
        for e in range(L):
            a, b = int(self.offsets[e]), int(self.offsets[e + 1])
            x[e, : b - a] = self.rows[a:b]
            m[e, : b - a] = self.meta[a:b]
        return x, m


def simulate_dispatch(cfg, world_size: int, xs: Sequence[torch.Tensor],
                      indices: Sequence[torch.Tensor]) -> List[RankDispatch]:
    """``dispatch`` of every rank (reference.py:68-148), all ranks in one process.

    The flat enumeration over ``(src_rank, t, k)`` is already the arrival order
    at every destination (source rank ascending, then the sender's ``(t, k)``
    order), so regrouping per global expert is one stable sort by expert id.
    """
    E, K = cfg.num_experts, cfg.experts_per_token
    L = E // world_size
    metas, srcs = [], []
    for r in range(world_size):
        idx = indices[r].to(torch.int64).cpu()
        n = idx.shape[0]
        t = torch.arange(n).repeat_interleave(K)
        k = torch.arange(K).repeat(n)
        e = idx.reshape(-1)
        metas.append(torch.stack([e, torch.full_like(e, r), t, k, torch.zeros_like(e)], dim=1))
        srcs.append(xs[r].cpu())
    meta = torch.cat(metas, 0)  # ordered by (src_rank, t, k)
    order = torch.sort(meta[:, 0], stable=True).indices  # -> (expert, src_rank, t, k)
    meta = meta[order]
    counts = torch.bincount(meta[:, 0], minlength=E)
    # gather the rows: row of pair = xs[src][t]
    base = torch.zeros(world_size + 1, dtype=torch.int64)
    base[1:] = torch.cumsum(torch.tensor([x.shape[0] for x in srcs]), 0)
    allx = torch.cat(srcs, 0)
    rows = allx[base[meta[:, 1]] + meta[:, 2]]
    out = []
    cum = torch.zeros(E + 1, dtype=torch.int64)
    cum[1:] = torch.cumsum(counts, 0)
    for d in range(world_size):
        a, b = int(cum[d * L]), int(cum[(d + 1) * L])
        out.append(RankDispatch(
            expert_num_tokens=counts[d * L:(d + 1) * L].to(torch.int32),
            rows=rows[a:b], meta=meta[a:b].to(torch.int32),
            offsets=(cum[d * L:(d + 1) * L + 1] - cum[d * L]).clone(),
        ))
    return out


def simulate_combine(cfg, world_size: int, disp: Sequence[RankDispatch], weights: Sequence[torch.Tensor],
                     num_tokens: Sequence[int], expert_scale=None) -> List[torch.Tensor]:
    """Expert placeholder + ``combine`` of every rank (reference.py:262, :151-234).

    Arrival order at the home rank is expert rank ascending, then local expert,
    then slot -- i.e. ascending global expert id, and within one expert the rows
    of different tokens never meet.  So each token's K contributions are added
    in ascending order of their global expert id, each add rounded to
    ``out_dtype``; that is K vectorised steps over all tokens.

    ``expert_scale`` (optional, tensor [num_experts] fp32) replaces the placeholder's
    ``1 + rank`` by a per-expert factor: a stand-in for a real expert op when the
    expert hook of the library is tested.
    """
    H = cfg.hidden_dim
    ys = [torch.zeros(n, H, dtype=cfg.out_dtype) for n in num_tokens]
    # per home rank, collect contributions in arrival order
    per_home_rows = [[] for _ in range(world_size)]
    per_home_meta = [[] for _ in range(world_size)]
    for d in range(world_size):
        if expert_scale is None:
            y = (disp[d].rows.to(cfg.out_dtype).to(torch.float32) * float(1 + d)).to(cfg.out_dtype)  # :262
        else:
            f = expert_scale.to(torch.float32)[disp[d].meta[:, 0].to(torch.int64)]
            y = (disp[d].rows.to(cfg.out_dtype).to(torch.float32) * f[:, None]).to(cfg.out_dtype)
        src = disp[d].meta[:, 1].to(torch.int64)
        for h in range(world_size):
            sel = (src == h).nonzero(as_tuple=True)[0]
            per_home_rows[h].append(y[sel])
            per_home_meta[h].append(disp[d].meta[sel])
    for h in range(world_size):
        rows = torch.cat(per_home_rows[h], 0)
        meta = torch.cat(per_home_meta[h], 0).to(torch.int64)
        t, k = meta[:, 2], meta[:, 3]
        w = weights[h].cpu().to(torch.float32)[t, k]
        contrib = rows.to(torch.float32) * w[:, None]
        # position of each arrival among the arrivals of its token (arrival order kept)
        order = torch.sort(t, stable=True).indices
        ts = t[order]
        first = torch.ones_like(ts, dtype=torch.bool)
        first[1:] = ts[1:] != ts[:-1]
        start = torch.where(first, torch.arange(ts.numel()), torch.zeros_like(ts))
        start = torch.cummax(start, 0).values
        step = torch.arange(ts.numel()) - start
        acc = ys[h]
        for s in range(int(step.max().item()) + 1 if step.numel() else 0):
            sel = order[step == s]
            tt = t[sel]
            acc[tt] = (acc[tt].to(torch.float32) + contrib[sel]).to(cfg.out_dtype)  # :232
    return ys


def simulate(cfg, world_size: int, rank_datas, expert_scale=None) -> "tuple[List[RankDispatch], List[torch.Tensor]]":
    """``ref_kernel`` (reference.py:256-272) for every rank: dispatch results and outputs."""
    xs = [rd.x.cpu() for rd in rank_datas]
    idx = [rd.indices.cpu() for rd in rank_datas]
    disp = simulate_dispatch(cfg, world_size, xs, idx)
    ys = simulate_combine(cfg, world_size, disp, [rd.weights for rd in rank_datas],
                          [rd.num_tokens for rd in rank_datas], expert_scale)
    return disp, ys


# --------------------------------------------------------------------------
# FP8 payload (no counterpart in the reference: parity unpinned upstream, the
# convention is fixed here and by the tests of this repository)
# --------------------------------------------------------------------------
FP8_BLOCK = 128
FP8_MAX = 448.0  # largest finite float8_e4m3fn


def fp8_quantise(x: torch.Tensor):
    """Per-128-element block: ``scale = amax / 448`` (fp32, 1.0 for an all-zero block),
    ``q = float8_e4m3fn(x / scale)`` (round to nearest even, saturating)."""
    n, H = x.shape
    blk = x.to(torch.float32).view(n, H // FP8_BLOCK, FP8_BLOCK)
    amax = blk.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (blk / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(n, H), scale.view(n, H // FP8_BLOCK)


def fp8_dequantise(q: torch.Tensor, scale: torch.Tensor, dtype) -> torch.Tensor:
    """``dtype(float(q) * scale)`` per block, one rounding."""
    n, H = q.shape
    blk = q.to(torch.float32).view(n, H // FP8_BLOCK, FP8_BLOCK) * scale[:, :, None]
    return blk.view(n, H).to(dtype)


# --------------------------------------------------------------------------
# comparators
# --------------------------------------------------------------------------
def dispatch_multiset(expert_num_tokens, rows_of_expert, meta_of_expert):
    """Key every received row by ``(local_expert, src_rank, token, k)`` -> raw row bytes.

    ``rows_of_expert(e)`` / ``meta_of_expert(e)`` return the valid rows / meta of
    local expert ``e``.  Two dispatch results are equal as multisets iff the
    returned dicts are equal.
    """
    out = {}
    for e, n in enumerate([int(v) for v in expert_num_tokens]):
        rows = rows_of_expert(e)[:n].contiguous()
        meta = meta_of_expert(e)[:n]
        raw = rows.view(torch.int16) if rows.element_size() == 2 else rows.view(torch.int8)
        for j in range(n):
            key = (e, int(meta[j, 1]), int(meta[j, 2]), int(meta[j, 3]))
            if key in out:
                raise AssertionError(f"duplicate row key {key}")
            out[key] = raw[j].numpy().tobytes()
    return out


def route_tables(indices: torch.Tensor, num_experts: int):
    """Host restatement of routing for one source rank: ``slot[t, k]`` = number of
    earlier pairs (in ``for t: for k`` order, reference.py:79-80) with the same expert,
    and the per-expert pair counts.  Literal loop; small inputs only."""
    idx = indices.cpu().tolist()
    seen = [0] * num_experts
    slots = []
    for experts in idx:
        row = []
        for e in experts:
            row.append(seen[e])
            seen[e] += 1
        slots.append(row)
    n_k = indices.shape[1] if indices.dim() == 2 else 0
    return (torch.tensor(slots, dtype=torch.int32).reshape(len(idx), n_k),
            torch.tensor(seen, dtype=torch.int32))
