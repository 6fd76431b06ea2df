"""The FP8 wire convention of the dispatch payload, frozen in tests/golden/fp8_quantiser.npz.

The reference has no FP8 path (parity for this payload is unpinned upstream); what is pinned here
is this repository's own convention: the golden file, an independent integer restatement of e4m3
round-to-nearest-even encoding, the CPU checker, and -- on a GPU -- the kernels."""
import os

import numpy as np
import pytest
import torch

from oracle import a2a_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fp8_quantiser.npz")
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    """float8_e4m3fn -> float32 from the bit fields: 1 sign, 4 exponent (bias 7), 3 mantissa;
    exponent 0 is subnormal (mantissa * 2^-9); 0x7f / 0xff are NaN (never produced)."""
    code = code.astype(np.int64)
    sign = np.where(code & 0x80, -1.0, 1.0)
    e, m = (code >> 3) & 0xF, code & 0x7
    mag = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    return (sign * mag).astype(np.float32)


def e4m3_encode(v: np.ndarray) -> np.ndarray:
    """float32 -> float8_e4m3fn, round to nearest even, saturating at +-448; integer arithmetic on
    the exactly scaled value (v * 2^9 is exact in float64 for every float32 in range)."""
    v = v.astype(np.float64)
    sign = np.where(np.signbit(v), 0x80, 0)
    a = np.minimum(np.abs(v), 448.0)
    out = np.zeros(v.shape, dtype=np.int64)
    sub = a < 2.0 ** -6
    # subnormal range: steps of 2^-9; a result of 8 steps is the smallest normal (code 0x08)
    q = a[sub] * 2.0 ** 9
    fl = np.floor(q)
    r = q - fl
    up = (r > 0.5) | ((r == 0.5) & (fl % 2 == 1))
    out[sub] = (fl + up).astype(np.int64)
    mant, ex = np.frexp(a[~sub])          # a = mant * 2^ex, mant in [0.5, 1)
    e = ex - 1                            # a = (2 * mant) * 2^e, 2*mant in [1, 2)
    q = (2.0 * mant - 1.0) * 8.0
    fl = np.floor(q)
    r = q - fl
    up = (r > 0.5) | ((r == 0.5) & (fl % 2 == 1))
    m = (fl + up).astype(np.int64)
    e = e + (m == 8)
    m = np.where(m == 8, 0, m)
    out[~sub] = np.minimum(((e + 7) << 3) | m, 0x7E)
    return (out | sign).astype(np.uint8)


def _load(name):
    z = np.load(GOLDEN)
    dt = DTYPES[name]
    x = torch.from_numpy(z[f"{name}_x"].view(np.int16).copy()).view(dt)
    back = torch.from_numpy(z[f"{name}_back"].view(np.int16).copy()).view(dt)
    return x, z[f"{name}_q"], z[f"{name}_scale"], back


def test_decode_table_agrees_with_torch():
    codes = np.arange(256, dtype=np.uint8)
    ok = (codes & 0x7F) != 0x7F
    t = torch.from_numpy(codes.copy()).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    assert np.array_equal(e4m3_decode(codes)[ok], t[ok])
    assert e4m3_decode(np.array([0x7E]))[0] == 448.0 and e4m3_decode(np.array([0x38]))[0] == 1.0
    assert e4m3_decode(np.array([0x01]))[0] == 2.0 ** -9 and e4m3_decode(np.array([0x08]))[0] == 2.0 ** -6


def test_known_answers_of_the_encoder():
    v = np.array([448.0, 1000.0, 1.0, 1.0625, 1.1875, 17.0, 19.0, 0.0, 2.0 ** -10, 3 * 2.0 ** -10, -2.0 ** -6], np.float32)
    want = np.array([0x7E, 0x7E, 0x38, 0x38, 0x3A, 0x58, 0x5A, 0x00, 0x00, 0x02, 0x88], np.uint8)
    #                max   sat   1.0  tie->even(1.0) tie->even(1.25) 17->16 19->20  0   half step->0  1.5 steps->2
    assert np.array_equal(e4m3_encode(v), want)
    t = torch.from_numpy(v).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(t, want)


@pytest.mark.parametrize("name", ["bf16", "fp16"])
def test_checker_reproduces_the_golden_file(name):
    x, q, scale, back = _load(name)
    gq, gs = O.fp8_quantise(x)
    assert np.array_equal(gq.view(torch.uint8).numpy(), q)
    assert np.array_equal(gs.numpy(), scale)
    assert torch.equal(O.fp8_dequantise(gq, gs, x.dtype).view(torch.int16), back.view(torch.int16))


@pytest.mark.parametrize("name", ["bf16", "fp16"])
def test_golden_file_follows_the_stated_convention(name):
    """scale = amax/448 in fp32 (1 for a zero block); q = e4m3(x/scale) by the integer encoder;
    back = dtype(decode(q) * scale)."""
    x, q, scale, back = _load(name)
    xf = x.to(torch.float32).numpy().reshape(x.shape[0], -1, 128)
    amax = np.abs(xf).max(-1)
    want_scale = np.where(amax > 0, (amax / np.float32(448.0)).astype(np.float32), np.float32(1.0))
    assert np.array_equal(want_scale, scale)
    ratio = (xf / scale[:, :, None]).astype(np.float32)
    assert np.array_equal(e4m3_encode(ratio).reshape(q.shape), q)
    deq = (e4m3_decode(q).reshape(xf.shape) * scale[:, :, None]).astype(np.float32).reshape(x.shape)
    assert torch.equal(torch.from_numpy(deq).to(x.dtype).view(torch.int16), back.view(torch.int16))
    assert int((scale == 1.0).sum()) >= 2  # the all-zero blocks are in the file


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["bf16", "fp16"])
def test_kernels_deliver_the_golden_rows(name):
    """Dispatch with the FP8 payload: what the expert rank holds is the golden file's dequantised row,
    bit for bit (one token per row of the file, two ranks stepped on one GPU, every row crosses the wire)."""
    import gpu_mode_kernels_b200 as pkg
    from gpu_mode_kernels_b200.local_world import LocalWorld

    x, _, _, back = _load(name)
    T, H = x.shape
    ws, E = 2, 4
    cfg = pkg.MoEConfig(E, 1, H, T, x.dtype, x.dtype)
    world = LocalWorld(cfg, ws, payload="fp8")
    try:
        rds = []
        for r in range(ws):
            rd = object.__new__(pkg.RankTestData)
            rd.num_tokens = T
            rd.x = x.to("cuda:0")
            # every token of rank r goes to an expert of the OTHER rank
            rd.indices = ((torch.arange(T, dtype=torch.int32) % 2) + 2 * (1 - r)).view(T, 1).to("cuda:0")
            rd.weights = torch.ones(T, 1, device="cuda:0")
            rds.append(rd)
        world.dispatch(rds)
        for r, c in enumerate(world.ctxs):
            counts, rows, meta = c.export_dispatch()
            torch.cuda.synchronize()
            n = counts.cpu().tolist()
            assert sum(n) == T
            for e in range(len(n)):
                tok = meta[e, : n[e], 2].cpu().long()
                assert torch.equal(rows[e, : n[e]].cpu().view(torch.int16), back[tok].view(torch.int16))
        world.check()
    finally:
        world.close()
