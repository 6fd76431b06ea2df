"""The CPU checker (oracle/) against golden vectors recorded from the reference itself."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

import gpu_mode_kernels_b200 as pkg
from oracle import a2a_oracle as O
from conftest import Golden


def test_generator_reproduces_golden_inputs(golden):
    """The seeded CPU generator yields the bytes the golden outputs were computed from."""
    kw = dict(golden.gen_kwargs)
    kw.pop("dtype", None)
    for r in range(golden.ws):
        _, rd, _, _ = pkg.generate_input(rank=r, world_size=golden.ws, dtype=golden.dtype, **kw)
        g = golden.rank_data(r)
        assert rd.num_tokens == g.num_tokens
        assert torch.equal(rd.indices, g.indices)
        assert torch.equal(rd.weights, g.weights)
        assert torch.equal(rd.x.view(torch.int16), g.x.view(torch.int16))


def test_simulate_matches_reference(golden):
    """Vectorised all-ranks oracle == reference, bit for bit (dispatch order included, and y)."""
    rds = [golden.rank_data(r) for r in range(golden.ws)]
    disp, ys = O.simulate(golden.cfg, golden.ws, rds)
    for r in range(golden.ws):
        n, rows, meta = golden.expected_dispatch(r)
        assert torch.equal(disp[r].expert_num_tokens, n)
        assert torch.equal(disp[r].meta, meta)
        assert torch.equal(disp[r].rows.view(torch.int16), rows.view(torch.int16))
        assert torch.equal(ys[r].view(torch.int16), golden.expected_y(r).view(torch.int16))


def _port_worker(rank, ws, name, port, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        g = Golden(name)
        rd = g.rank_data(rank)
        ata = O.PortAllToAll(g.cfg, rank, ws)
        n, ex, em = ata.dispatch(rd.x, rd.indices)
        en, rows, meta = g.expected_dispatch(rank)
        ok = torch.equal(n, en)
        got_rows = torch.cat([ex[e, : int(n[e])] for e in range(n.numel())], 0)
        got_meta = torch.cat([em[e, : int(n[e])] for e in range(n.numel())], 0)
        ok = ok and torch.equal(got_rows.view(torch.int16), rows.view(torch.int16)) and torch.equal(got_meta, meta)
        y = O.port_ref_kernel((g.cfg, rd, rank, ws))
        ok = ok and torch.equal(y.view(torch.int16), g.expected_y(rank).view(torch.int16))
        y2 = O.port_ref_kernel((g.cfg, rd, rank, ws), valid_rows_only=True)
        ok = ok and torch.equal(y2.view(torch.int16), g.expected_y(rank).view(torch.int16))
        q.put((rank, bool(ok)))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("name,port", [("c1_ws2_bf16", 29701), ("ws2_fp16_task", 29702)])
def test_port_under_gloo_matches_reference(name, port):
    """The literal per-rank port, two CPU ranks on gloo, == reference bit for bit."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_port_worker, args=(r, 2, name, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
    assert res == {0: True, 1: True}


def test_fp8_roundtrip_convention():
    """Quantiser convention: scale = amax/448 per 128 block; zero blocks get scale 1; error bounded."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(7, 512, generator=g).to(torch.bfloat16)
    x[3, 128:256] = 0
    q, s = O.fp8_quantise(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (7, 4)
    assert s[3, 1].item() == 1.0
    amax = x.float().view(7, 4, 128).abs().amax(-1)
    assert torch.equal(torch.where(amax > 0, amax / 448.0, torch.ones_like(amax)), s)
    dq = O.fp8_dequantise(q, s, torch.bfloat16)
    assert torch.equal(dq[3, 128:256], torch.zeros(128, dtype=torch.bfloat16))
    # e4m3 has 3 mantissa bits: relative step 2^-3 at worst -> half-step error 2^-4 of the block max
    err = (dq.float() - x.float()).abs().view(7, 4, 128).amax(-1)
    assert bool((err <= amax * 2 ** -4 + 1e-6).all())
