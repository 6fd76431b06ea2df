"""The dispatch digests bench.py and the harness use to prove a bit-exact dispatch on many ranks
without shipping the rows: equal inputs give equal digests; a changed count, a flipped bit, two
swapped rows or two swapped records change them."""
import torch

import gpu_mode_kernels_b200 as pkg
from gpu_mode_kernels_b200 import verify
from oracle import a2a_oracle as O


def _dispatch():
    ws = 2
    datas = [pkg.workload_input("c1", r, ws) for r in range(ws)]
    disp, _ = O.simulate(datas[0][0], ws, [d[1] for d in datas])
    return disp[0]


def test_digest_is_reproducible_and_sensitive():
    d = _dispatch()
    base = verify.dispatch_digest(d.expert_num_tokens, d.rows, d.meta)
    assert base == verify.dispatch_digest(d.expert_num_tokens.clone(), d.rows.clone(), d.meta.clone())
    counts = d.expert_num_tokens.clone()
    counts[0] += 1
    assert verify.dispatch_digest(counts, d.rows, d.meta)[0] != base[0]
    rows = d.rows.clone()
    rows.view(torch.int16)[3, 5] ^= 1  # one bit of one element
    assert verify.dispatch_digest(d.expert_num_tokens, rows, d.meta)[1] != base[1]
    rows = d.rows.clone()
    rows[[0, 1]] = rows[[1, 0]]  # same multiset, other order
    if not torch.equal(rows[0], rows[1]):
        assert verify.dispatch_digest(d.expert_num_tokens, rows, d.meta)[1] != base[1]
    meta = d.meta.clone()
    meta[[0, 1]] = meta[[1, 0]]
    assert verify.dispatch_digest(d.expert_num_tokens, d.rows, meta)[2] != base[2]


def test_compact_dispatch_takes_the_valid_prefixes():
    counts = torch.tensor([2, 0, 1], dtype=torch.int32)
    rows = torch.arange(3 * 4 * 8, dtype=torch.float32).view(3, 4, 8).to(torch.bfloat16)
    meta = torch.arange(3 * 4 * 5, dtype=torch.int32).view(3, 4, 5)
    r, m = verify.compact_dispatch(counts, rows, meta)
    assert r.shape == (3, 8) and m.shape == (3, 5)
    assert torch.equal(r[2], rows[2, 0]) and torch.equal(m[1], meta[0, 1])
    r0, m0 = verify.compact_dispatch(torch.zeros(3, dtype=torch.int32), rows, meta)
    assert r0.shape[0] == 0 and m0.shape[0] == 0
    assert verify.dispatch_digest(torch.zeros(3, dtype=torch.int32), r0, m0)[1:] == (0, 0)
