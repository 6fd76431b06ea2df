import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """One golden case recorded from the reference (see tests/golden/make_golden.py)."""

    def __init__(self, name):
        import gpu_mode_kernels_b200 as pkg

        z = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"))
        self.name = name
        self.ws = int(z["world_size"])
        kw = {k[4:]: z[k].item() for k in z.files if k.startswith("cfg_")}
        self.gen_kwargs = dict(kw)
        self.dtype = getattr(torch, kw.pop("dtype", "bfloat16"))
        self.cfg = pkg.MoEConfig(kw["num_experts"], kw["experts_per_token"], kw["hidden_dim"],
                                 kw["max_num_tokens"], self.dtype, self.dtype)
        self.z = z

    def f16(self, key):
        a = self.z[key]
        return torch.from_numpy(a.view(np.int16).copy()).view(self.dtype)

    def rank_data(self, r):
        import gpu_mode_kernels_b200 as pkg

        rd = object.__new__(pkg.RankTestData)
        rd.num_tokens = int(self.z[f"r{r}_num_tokens"])
        rd.indices = torch.from_numpy(self.z[f"r{r}_indices"].copy())
        rd.weights = torch.from_numpy(self.z[f"r{r}_weights"].copy())
        rd.x = self.f16(f"r{r}_x")
        return rd

    def expected_dispatch(self, r):
        n = torch.from_numpy(self.z[f"r{r}_expert_num_tokens"].copy())
        rows = self.f16(f"r{r}_rows")
        meta = torch.from_numpy(self.z[f"r{r}_meta"].copy())
        return n, rows, meta

    def expected_y(self, r):
        return self.f16(f"r{r}_y")


GOLDEN_NAMES = ["c1_ws2_bf16", "ws1_bf16", "ws4_bf16_ragged", "ws8_bf16_zipf", "ws2_fp16_task", "ws8_fp16_task"]


@pytest.fixture(params=GOLDEN_NAMES)
def golden(request):
    return Golden(request.param)
