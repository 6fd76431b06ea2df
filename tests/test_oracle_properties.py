"""Property tests (CPU) tying the checker's pieces together on random small problems."""
import torch
from hypothesis import given, settings, strategies as st

import gpu_mode_kernels_b200 as pkg
from gpu_mode_kernels_b200 import traffic
from oracle import a2a_oracle as O


@st.composite
def problems(draw):
    ws = draw(st.sampled_from([1, 2, 4, 8]))
    L = draw(st.integers(1, 4))
    E = ws * L
    K = draw(st.integers(1, min(E, 6)))
    T = draw(st.integers(1, 12))
    seed = draw(st.integers(0, 10_000))
    return ws, E, K, T, seed


@settings(max_examples=40, deadline=None)
@given(problems())
def test_slots_are_positions_inside_each_source_contribution(p):
    """route_tables' slot of pair (t,k) == position of that row among the rows its source sent to the
    expert, in the order the reference delivers them (source rank ascending, then (t,k))."""
    ws, E, K, T, seed = p
    datas = [pkg.generate_input(E, K, 8, T, seed=seed, rank=r, world_size=ws, ragged=True) for r in range(ws)]
    cfg = datas[0][0]
    rds = [d[1] for d in datas]
    disp, ys = O.simulate(cfg, ws, rds)
    L = E // ws
    slots = [O.route_tables(rd.indices, E)[0] for rd in rds]
    total = 0
    for d in range(ws):
        n = disp[d].expert_num_tokens.tolist()
        off = disp[d].offsets.tolist()
        total += sum(n)
        for l in range(L):
            meta = disp[d].meta[off[l]:off[l + 1]]
            seen = {}
            for row in meta.tolist():
                e, src, t, k, _ = row
                assert e == d * L + l
                pos = seen.get(src, 0)
                assert int(slots[src][t, k]) == pos
                seen[src] = pos + 1
            assert sorted(seen) == list(seen)  # sources arrive in ascending order
    assert total == sum(rd.num_tokens for rd in rds) * K
    for r in range(ws):
        assert ys[r].shape == (rds[r].num_tokens, 8)


@settings(max_examples=40, deadline=None)
@given(problems())
def test_traffic_accounting_is_conservative(p):
    ws, E, K, T, seed = p
    idx = [pkg.generate_input(E, K, 8, T, seed=seed, rank=r, world_size=ws)[1].indices for r in range(ws)]
    pairs, rows = traffic.pair_counts(idx, E, ws)
    assert int(pairs.sum()) == ws * T * K
    assert bool((rows <= pairs).all()) and bool((rows <= T).all())
    s = traffic.summarize(idx, E, ws, 64)
    assert s["busiest_rows_dedup"] <= s["busiest_rows"] <= T * K * max(1, ws - 1)
    assert s["wire_bytes"] == s["algorithmic_bytes"]
    assert traffic.summarize(idx, E, ws, 64, "dedup")["wire_bytes"] <= s["wire_bytes"]


def test_combine_order_is_ascending_expert_with_per_step_rounding():
    """A hand-checkable case of the reference's accumulation (reference.py:226-232): contributions
    are added in ascending global-expert order, each add rounded to bf16."""
    cfg = pkg.MoEConfig(4, 3, 8, 1)
    rd = object.__new__(pkg.RankTestData)
    rd.num_tokens = 1
    rd.indices = torch.tensor([[3, 0, 2]], dtype=torch.int32)
    rd.weights = torch.tensor([[0.3, 0.5, 0.2]])
    rd.x = torch.full((1, 8), 1.0078125, dtype=torch.bfloat16)  # 1 + 2^-7, exactly representable
    _, ys = O.simulate(cfg, 1, [rd])
    acc = torch.zeros(8, dtype=torch.bfloat16)
    for e, w in sorted(zip([3, 0, 2], [0.3, 0.5, 0.2])):
        acc = (acc.float() + rd.x[0].float() * torch.tensor(w)).to(torch.bfloat16)
    assert torch.equal(ys[0][0], acc)
