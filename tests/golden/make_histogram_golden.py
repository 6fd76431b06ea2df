"""Write tests/golden/histogram.npz: inputs of this repository's CPU generator (the reference's recipe,
pmpp_v2/histogram_py/reference.py:22-45, on a CPU generator) and the counts the reference's own
operator call gives for them -- ``torch.bincount(data, minlength=256)`` (reference.py:17), executed
here on the CPU.

    python tests/golden/make_histogram_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import histogram_oracle as HO  # noqa: E402

CASES = [(5120, 9991, 10), (7840, 2105, 10), (30080, 4254, 90), (1000, 3, 100), (4099, 17, 40)]


def main():
    out = {"cases": np.int64(len(CASES))}
    for i, (size, seed, contention) in enumerate(CASES):
        data, _ = HO.generate_input(size, contention, seed)
        out[f"c{i}_spec"] = np.array([size, seed, contention], dtype=np.int64)
        out[f"c{i}_data"] = data.numpy()
        out[f"c{i}_hist"] = torch.bincount(data, minlength=256).numpy()  # the reference's call
    path = os.path.join(HERE, "histogram.npz")
    np.savez_compressed(path, **out)
    print(path)


if __name__ == "__main__":
    main()
