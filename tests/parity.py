"""Parity policy shared by the GPU tests: tolerances and the FP8 rules."""
import torch

from oracle import a2a_oracle as O


def tol(dtype, payload="direct"):
    """Combine tolerance: rtol=atol=2e-2 in bf16 (6e-2 with the FP8 payload); fp16 runs
    are held to the reference task's own rtol=1e-2, atol=5e-3 (reference.py:279)."""
    if payload == "fp8":
        return dict(rtol=6e-2, atol=6e-2)
    if dtype == torch.float16:
        return dict(rtol=1e-2, atol=5e-3)
    return dict(rtol=2e-2, atol=2e-2)


def quantised_inputs(rds, dtype):
    """The same rank inputs with x replaced by what the FP8 wire format delivers."""
    out = []
    for rd in rds:
        q = rd.to("cpu")
        q.x = fp8_roundtrip(q.x, dtype)
        out.append(q)
    return out


def check_y(cfg, ws, rds_cpu, out, ys, payload, ranks=None):
    """Combine parity.  bf16/fp16 payloads: every element within the stated tolerance of the
    reference.  FP8 payload: (a) every element within rtol=atol=2e-2 of the checker run on the
    dequantised inputs (isolates the kernels from the format), and (b) against the bf16
    reference at rtol=atol=6e-2.  e4m3 alone has a worst-case relative error of 1/17 = 5.9 %, and
    the reference's own per-add bf16 rounding moves it by about another per cent, so a few
    elements in 10^5 land up to ~1.2x outside 6e-2 whatever the kernel does; (b) therefore
    allows a 1e-4 fraction of elements up to 1.25x the tolerance and nothing beyond."""
    dtype = cfg.in_dtype
    ranks = range(ws) if ranks is None else ranks
    if payload != "fp8":
        for r in ranks:
            torch.testing.assert_close(out[r].cpu().float(), ys[r].float(), **tol(dtype, payload))
        return
    _, ys_q = O.simulate(cfg, ws, quantised_inputs(rds_cpu, dtype))
    t = tol(dtype, "fp8")
    for r in ranks:
        got = out[r].cpu().float()
        torch.testing.assert_close(got, ys_q[r].float(), **tol(dtype, "direct"))
        diff = (got - ys[r].float()).abs()
        allowed = t["atol"] + t["rtol"] * ys[r].float().abs()
        ratio = diff / allowed
        assert float(ratio.max()) <= 1.25, f"rank {r}: worst diff/tol {float(ratio.max()):.3f}"
        assert int((ratio > 1).sum()) <= max(1, int(1e-4 * ratio.numel())), f"rank {r}: {int((ratio > 1).sum())} outliers"


def fp8_roundtrip(rows, dtype):
    """What the receiver holds when the payload crossed the wire as e4m3 + per-128 scales."""
    q, s = O.fp8_quantise(rows)
    return O.fp8_dequantise(q, s, dtype)


