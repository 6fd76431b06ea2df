"""In-kernel trace -> chrome trace, merged over the ranks, with wait histograms.

The kernels stamp, per block, the SM cycle counter at every phase boundary
(``a2a_trace_enable`` / ``a2a_trace_read``); this module turns the stamps of one traced launch
per rank into events, merges the ranks on rank 0 and writes one JSON file that
``chrome://tracing`` / Perfetto open: one process per rank, one thread per block.  It plays the
part of the profile post-processing of the reference's last submission
(amd-distributed/all2all/submission_v9.py:985-1026: per-rank event lists gathered to rank 0
and dumped as a chrome trace), plus what that code lacks: per-(phase, peer) histograms of how
long blocks sat waiting for a flag.

Stamp layout (int64 ``[blocks, 32]``): 0 global timer in ns at the block's start, 1 start,
2 routing done (pipelined kernel: the block's role bits), 3 sending / routing done, 4 first
dispatch flag seen, 5 expert pass done, 6 expert flags seen, 7 combine done; pipelined kernel
only: 8+i rows of the i-th source seen, 16+i done (sources in the order own rank, rank-1, ...),
24+i the block's stores to the i-th destination (rank+i) complete.  Slots 1.. are SM cycles;
a zero slot means "not stamped".  Times are reported relative to the earliest block start of the
same rank (the global timers of different GPUs are not synchronised; the ranks of a traced call
are aligned by the device-side rendezvous that precedes it).
"""
from __future__ import annotations

import json
from typing import Dict, List, Sequence

ROLE_SENDER, ROLE_EXPERT, ROLE_ROUTER, ROLE_WATCHER = 1, 2, 4, 8
WAIT_BUCKETS_US = (1, 2, 4, 8, 16, 32, 64, 1e9)


def _role_name(bits: int) -> str:
    names = [n for b, n in ((ROLE_SENDER, "sender"), (ROLE_ROUTER, "router"), (ROLE_EXPERT, "expert"),
                            (ROLE_WATCHER, "watcher")) if bits & b]
    return "+".join(names) or "block"


def rank_events(stamps, rank: int, *, sm_mhz: float, world_size: int = 0, pipelined: bool = None) -> Dict:
    """Events of one rank from its stamp table (a tensor or nested list ``[blocks][32]``).

    Returns ``{"rank", "events": [{"name","cat","block","ts","dur","peer"}], "marks": {...}}`` with
    times in microseconds relative to the rank's earliest block start."""
    rows = stamps.tolist() if hasattr(stamps, "tolist") else [list(r) for r in stamps]
    rows = [r for r in rows if r[1] != 0]
    if not rows:
        return {"rank": rank, "events": [], "blocks": 0}
    t0 = min(r[0] for r in rows)
    if pipelined is None:
        pipelined = any(0 < r[2] < 16 for r in rows)  # role bits, not a cycle count
    cyc_us = 1.0 / float(sm_mhz)

    events: List[Dict] = []

    def at(r, slot):
        """Microseconds since t0 of stamp `slot` of block row r, or None."""
        return None if r[slot] == 0 else (r[0] - t0) * 1e-3 + (r[slot] - r[1]) * cyc_us

    def add(block, name, cat, a, b, peer=-1):
        if a is not None and b is not None and b >= a:
            events.append({"name": name, "cat": cat, "block": block, "ts": a, "dur": b - a, "peer": peer})

    for b, r in enumerate(rows):
        start = at(r, 1)
        if not pipelined:
            add(b, "route", "work", start, at(r, 2))
            add(b, "send", "work", at(r, 2), at(r, 3))
            add(b, "wait dispatch", "wait", at(r, 3), at(r, 4))
            add(b, "expert", "work", at(r, 4), at(r, 5))
            add(b, "wait experts", "wait", at(r, 5), at(r, 6))
            add(b, "combine", "work", at(r, 6), at(r, 7))
            continue
        role = int(r[2])
        prev = start
        if role & ROLE_SENDER:
            n = world_size or 9
            for i in range(1, min(n, 8)):
                t = at(r, 24 + i)
                if t is not None:
                    add(b, f"send to +{i}", "work", prev, t, peer=(rank + i) % world_size if world_size else i)
                    prev = t
            add(b, "drain", "work", prev, at(r, 3))
            prev = at(r, 3) or prev
        if role & ROLE_ROUTER:
            add(b, "route", "work", start, at(r, 3))
            prev = at(r, 3) or prev
        if role & ROLE_EXPERT:
            for i in range(8):
                seen, done = at(r, 8 + i), at(r, 16 + i)
                if seen is None:
                    break
                peer = (rank - i) % world_size if world_size else i
                add(b, f"wait rows of -{i}", "wait", prev, seen, peer=peer)
                add(b, f"expert rows of -{i}", "work", seen, done, peer=peer)
                prev = done if done is not None else seen
        add(b, "wait partials" if role else "wait", "wait", at(r, 5), at(r, 6))
        add(b, "combine", "work", at(r, 6), at(r, 7))
    for e in events:
        e["role"] = _role_name(int(rows[e["block"]][2])) if pipelined else "block"
    return {"rank": rank, "events": events, "blocks": len(rows), "pipelined": bool(pipelined)}


def wait_histograms(per_rank: Sequence[Dict]) -> Dict[str, List[int]]:
    """Counts of wait durations per (event name) over all ranks and blocks, in WAIT_BUCKETS_US bins."""
    hist: Dict[str, List[int]] = {}
    for pr in per_rank:
        for e in pr["events"]:
            if e["cat"] != "wait":
                continue
            h = hist.setdefault(e["name"], [0] * len(WAIT_BUCKETS_US))
            for i, edge in enumerate(WAIT_BUCKETS_US):
                if e["dur"] < edge:
                    h[i] += 1
                    break
    return hist


def write_chrome_trace(path: str, per_rank: Sequence[Dict]) -> None:
    """One JSON file for chrome://tracing / Perfetto: pid = rank, tid = block."""
    out = []
    for pr in per_rank:
        out.append({"name": "process_name", "ph": "M", "pid": pr["rank"], "args": {"name": f"rank {pr['rank']}"}})
        for e in pr["events"]:
            out.append({"name": e["name"], "cat": e["cat"], "ph": "X", "pid": pr["rank"], "tid": e["block"],
                        "ts": round(e["ts"], 3), "dur": round(e["dur"], 3), "args": {"peer": e["peer"], "role": e["role"]}})
    with open(path, "w") as f:
        json.dump({"traceEvents": out, "displayTimeUnit": "ns"}, f)


def summarize(per_rank: Sequence[Dict]) -> str:
    """Phase table per rank (when the first / last block began and ended each kind of event,
    microseconds from the rank's first block start) and the wait histograms."""
    lines = []
    for pr in per_rank:
        lines.append(f"rank {pr['rank']}: {pr['blocks']} blocks")
        groups: Dict[str, List[Dict]] = {}
        for e in pr["events"]:
            groups.setdefault(e["name"], []).append(e)
        lines.append(f"  {'event':<22}{'blocks':>7}{'first start':>13}{'last end':>10}{'median dur':>12}{'max dur':>9}")
        for name, es in sorted(groups.items(), key=lambda kv: min(e["ts"] for e in kv[1])):
            durs = sorted(e["dur"] for e in es)
            lines.append(f"  {name:<22}{len(es):>7}{min(e['ts'] for e in es):>13.1f}{max(e['ts'] + e['dur'] for e in es):>10.1f}"
                         f"{durs[len(durs) // 2]:>12.1f}{durs[-1]:>9.1f}")
    lines.append("wait histograms (all ranks, all blocks); bins < " +
                 ", ".join("inf" if b > 1e8 else f"{b:g}" for b in WAIT_BUCKETS_US) + " us")
    for name, h in sorted(wait_histograms(per_rank).items()):
        lines.append(f"  {name:<22}" + " ".join(f"{c:>6}" for c in h))
    return "\n".join(lines) + "\n"
