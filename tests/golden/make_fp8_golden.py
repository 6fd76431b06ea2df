"""Freeze the FP8 wire convention of the dispatch payload in a golden file.

    python tests/golden/make_fp8_golden.py

The reference has no FP8 path, so there is nothing upstream to record: this script runs the
checker's quantiser (oracle/a2a_oracle.py: per 128 values ``scale = amax / 448`` -- 1 for an
all-zero block --, ``q = e4m3(x / scale)`` round-to-nearest-even saturating, receiver stores
``dtype(float(q) * scale)``) on inputs that hit its corner cases and writes inputs, e4m3 bytes,
scales and dequantised rows to ``fp8_quantiser.npz``.  From then on the file, not the code,
defines the convention: the CPU tests hold the checker to it and to an independent integer
restatement of e4m3 rounding, the GPU tests hold the kernels to it.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import a2a_oracle as O  # noqa: E402

H = 512  # four scale blocks per row


def inputs(dtype):
    g = torch.Generator().manual_seed(2024)
    rows = [torch.randn(24, H, generator=g)]                       # the benchmark's distribution
    rows.append(torch.randn(4, H, generator=g) * 1e-3)             # small magnitudes
    rows.append(torch.randn(4, H, generator=g) * 300.0)            # large magnitudes
    z = torch.randn(2, H, generator=g)
    z[:, 128:256] = 0.0                                            # an all-zero block: scale 1
    rows.append(z)
    one = torch.zeros(2, H)
    one[0, 5], one[1, 300] = 3.0, -7.5                             # a block with a single non-zero value
    rows.append(one)
    ties = torch.zeros(2, H)
    # amax 448 -> scale 1: values halfway between two e4m3 codes round to even
    ties[0, :16] = torch.tensor([448.0, 17.0, 19.0, 21.0, 23.0, 25.0, 27.0, 29.0, 31.0, 1.0625, 1.1875, 0.001, 0.002,
                                 0.0009765625, 0.0029296875, -0.0048828125])
    ties[1, 128:144] = -ties[0, :16]
    rows.append(ties)
    return torch.cat(rows).to(dtype)


def main():
    out = {}
    for name, dtype in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        x = inputs(dtype)
        q, scale = O.fp8_quantise(x)
        back = O.fp8_dequantise(q, scale, dtype)
        out[f"{name}_x"] = x.view(torch.int16).numpy().view(np.uint16)
        out[f"{name}_q"] = q.view(torch.uint8).numpy()
        out[f"{name}_scale"] = scale.numpy()
        out[f"{name}_back"] = back.view(torch.int16).numpy().view(np.uint16)
    path = os.path.join(HERE, "fp8_quantiser.npz")
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
