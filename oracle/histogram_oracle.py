"""CPU checker of the 256-bin byte histogram (test infrastructure; never on a product path).

The reference's whole algorithm is one call, ``torch.bincount(data, minlength=256)`` on a uint8
tensor into an int64 output (pmpp_v2/histogram_py/reference.py:6-19) -- a PyTorch operator, and
PyTorch is installed here, so ``ref_histogram`` makes that very call on the CPU.  ``count_bytes``
restates it without the operator (numpy integer arithmetic) so that the two can be held against
each other and against hand-written answers.  Parity is pinned by the reference's own call executed
here; the reference's ``generate_input`` needs a CUDA generator (reference.py:22-45), so
``generate_input`` below follows its recipe on a CPU generator: uniform bytes, then one "evil" value
written over a ``contention`` per cent fraction of the positions.
"""
from __future__ import annotations

import numpy as np
import torch

NUM_BINS = 256


def ref_histogram(data: torch.Tensor) -> torch.Tensor:
    """reference.py:17: ``torch.bincount(data, minlength=256)`` (int64 [256])."""
    return torch.bincount(data.cpu().to(torch.int64), minlength=NUM_BINS)


def count_bytes(data) -> np.ndarray:
    """The same counts without bincount: one equality sum per bin."""
    a = np.asarray(data.cpu() if hasattr(data, "cpu") else data, dtype=np.uint8).reshape(-1)
    out = np.zeros(NUM_BINS, dtype=np.int64)
    for b in range(NUM_BINS):
        out[b] = int((a == b).sum())
    return out


def generate_input(size: int, contention: float, seed: int, device="cpu"):
    """(data uint8 [size], output int64 [256]) in the style of reference.py:22-45."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    data = torch.randint(0, 256, (size,), dtype=torch.uint8, generator=gen)
    evil_value = torch.randint(0, 256, (), dtype=torch.uint8, generator=gen)
    evil_loc = torch.rand((size,), dtype=torch.float32, generator=gen) < (contention / 100.0)
    data[evil_loc] = evil_value
    output = torch.empty(NUM_BINS, dtype=torch.int64, device=device)
    return data.contiguous().to(device), output


# The reference task's own test and benchmark cases (task.yml:26-39): (size, seed, contention)
REFERENCE_TESTS = [(5120, 9991, 10), (7840, 2105, 10), (30080, 9999, 10), (30080, 4254, 90), (100000, 1212, 10)]
REFERENCE_BENCHMARKS = [(1310720, 6252, 10), (2621440, 8841, 10), (2621440, 3411, 40), (2621440, 8753, 90),
                        (5242880, 6252, 10), (10485760, 8841, 10)]
