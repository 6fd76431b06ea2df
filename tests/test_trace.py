"""The in-kernel trace: conversion of stamp tables to events / chrome JSON / wait histograms on
synthetic stamps (CPU), and on a GPU that the stamps of a real launch are ordered and that a
launch with tracing off leaves the trace buffer untouched."""
import json

import pytest
import torch

from gpu_mode_kernels_b200 import trace as tracing


def _stamps():
    """Two ranks' worth of hand-made stamp rows of the pipelined kernel at 1000 MHz (1 cycle = 1 ns)."""
    s = torch.zeros(4, 32, dtype=torch.int64)
    # block 0: sender (+watcher): start at 5000 ns; destinations +1 and +2 finished 4 and 9 us later
    s[0, 0], s[0, 1], s[0, 2], s[0, 3] = 5000, 100, tracing.ROLE_SENDER | tracing.ROLE_WATCHER, 100 + 10000
    s[0, 25], s[0, 26] = 100 + 4000, 100 + 9000
    s[0, 5], s[0, 6], s[0, 7] = 100 + 10500, 100 + 30000, 100 + 33000
    # block 1: router + expert: routed after 2 us; own rows at 2.5 us (done 4), rows of -1 at 12 us (done 14)
    s[1, 0], s[1, 1], s[1, 2], s[1, 3] = 6000, 50, tracing.ROLE_EXPERT | tracing.ROLE_ROUTER, 50 + 2000
    s[1, 8], s[1, 16], s[1, 9], s[1, 17] = 50 + 2500, 50 + 4000, 50 + 12000, 50 + 14000
    s[1, 5], s[1, 6], s[1, 7] = 50 + 14100, 50 + 29000, 50 + 31000
    # block 2: expert only
    s[2, 0], s[2, 1], s[2, 2] = 5500, 70, tracing.ROLE_EXPERT
    s[2, 8], s[2, 16] = 70 + 3000, 70 + 5000
    # block 3: never ran (all zero)
    return s


def test_events_of_a_pipelined_launch():
    ev = tracing.rank_events(_stamps(), rank=1, sm_mhz=1000.0, world_size=3)
    assert ev["blocks"] == 3 and ev["pipelined"]
    by = {(e["block"], e["name"]): e for e in ev["events"]}
    # times are relative to the earliest block start (block 0 at 5000 ns)
    assert by[(0, "send to +1")]["ts"] == pytest.approx(0.0) and by[(0, "send to +1")]["dur"] == pytest.approx(4.0)
    assert by[(0, "send to +1")]["peer"] == 2 and by[(0, "send to +2")]["peer"] == 0
    assert by[(0, "send to +2")]["dur"] == pytest.approx(5.0)
    assert by[(0, "combine")]["dur"] == pytest.approx(3.0) and by[(0, "wait partials")]["dur"] == pytest.approx(19.5)
    assert by[(1, "route")]["ts"] == pytest.approx(1.0) and by[(1, "route")]["dur"] == pytest.approx(2.0)
    assert by[(1, "wait rows of -0")]["dur"] == pytest.approx(0.5) and by[(1, "wait rows of -0")]["peer"] == 1
    assert by[(1, "wait rows of -1")]["dur"] == pytest.approx(8.0) and by[(1, "wait rows of -1")]["peer"] == 0
    assert by[(1, "expert rows of -1")]["dur"] == pytest.approx(2.0)
    assert by[(2, "wait rows of -0")]["dur"] == pytest.approx(3.0)
    assert by[(0, "combine")]["role"] == "sender+watcher" and by[(1, "route")]["role"] == "router+expert"


def test_phased_stamps_chrome_json_and_histograms(tmp_path):
    s = torch.zeros(2, 32, dtype=torch.int64)
    for b in range(2):
        s[b, 0], s[b, 1] = 1000 + 100 * b, 10
        for slot, us in zip(range(2, 8), (3, 30, 35 + 10 * b, 48, 55, 90)):
            s[b, slot] = 10 + us * 2000  # 2000 MHz
    ranks = [tracing.rank_events(s, r, sm_mhz=2000.0, world_size=2) for r in range(2)]
    assert not ranks[0]["pipelined"]
    names = [e["name"] for e in ranks[0]["events"] if e["block"] == 0]
    assert names == ["route", "send", "wait dispatch", "expert", "wait experts", "combine"]
    hist = tracing.wait_histograms(ranks)
    assert sum(hist["wait dispatch"]) == 4 and sum(hist["wait experts"]) == 4
    assert hist["wait dispatch"][tracing.WAIT_BUCKETS_US.index(8)] == 2      # 5 us waits of block 0
    assert hist["wait dispatch"][tracing.WAIT_BUCKETS_US.index(16)] == 2     # 15 us waits of block 1
    path = tmp_path / "t.json"
    tracing.write_chrome_trace(str(path), ranks)
    doc = json.loads(path.read_text())
    xs = [e for e in doc["traceEvents"] if e["ph"] == "X"]
    assert len(xs) == 24 and {e["pid"] for e in xs} == {0, 1} and {e["tid"] for e in xs} == {0, 1}
    text = tracing.summarize(ranks)
    assert "rank 1: 2 blocks" in text and "wait histograms" in text and "combine" in text


def test_empty_trace():
    ev = tracing.rank_events(torch.zeros(5, 32, dtype=torch.int64), 0, sm_mhz=1965.0)
    assert ev["events"] == [] and ev["blocks"] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("schedule,combine", [("pipelined", "push"), ("pipelined", "pull"), ("phased", "pull")])
def test_stamps_of_a_real_launch_are_ordered_and_tracing_off_writes_nothing(schedule, combine):
    import gpu_mode_kernels_b200 as pkg
    from gpu_mode_kernels_b200.all2all import A2AContext

    cfg, rd, _, _ = pkg.workload_input("c2", 0, 1)
    d = rd.to("cuda:0")
    ctx = A2AContext(cfg, 0, 1, device=0, payload="dedup", schedule=schedule, combine=combine)
    try:
        ctx.trace_enable(True)
        ctx.forward(d.x, d.indices, d.weights)
        st = ctx.trace_read()
        assert st.shape[1] == 32 and st.shape[0] >= 148
        assert bool((st[:, 1] > 0).all()) and bool((st[:, 0] > 0).all())
        seq = [1, 5, 6, 7] if schedule == "pipelined" else [1, 2, 3, 4, 5, 6, 7]
        for a, b in zip(seq, seq[1:]):
            both = (st[:, a] > 0) & (st[:, b] > 0)  # a block without combine items never stamps "experts seen"
            assert bool(both.any()) and bool((st[both, a] <= st[both, b]).all()), (a, b)
        if schedule == "pipelined":
            experts = st[(st[:, 2] & tracing.ROLE_EXPERT) != 0]
            assert experts.shape[0] == st.shape[0]  # world size 1: no sender blocks
            assert bool((experts[:, 8] >= experts[:, 1]).all()) and bool((experts[:, 16] >= experts[:, 8]).all())
            assert 1 <= int(((st[:, 2] & tracing.ROLE_ROUTER) != 0).sum()) <= 8  # router blocks of the one destination
        ev = tracing.rank_events(st, 0, sm_mhz=1965.0, world_size=1)
        assert ev["blocks"] == st.shape[0] and len(ev["events"]) >= 3 * st.shape[0]
        assert all(0 <= e["ts"] < 1e4 and 0 <= e["dur"] < 1e4 for e in ev["events"])
        # tracing off: the next launch must leave the buffer as it is
        ctx.trace_enable(False)
        ctx.forward(d.x, d.indices, d.weights)
        torch.cuda.synchronize()
        assert torch.equal(ctx.trace_read(), st)
        ctx.check()
    finally:
        ctx.close()
