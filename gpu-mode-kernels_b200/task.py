"""Task contract of the MoE all-to-all path: config, per-rank inputs, workloads.

Mirrors the names and field meanings of the reference task so that a
``data = (cfg, rank_data, rank, world_size)`` tuple built here is accepted by
both the reference's ``ref_kernel`` and this package's ``custom_kernel``:

* ``MoEConfig``      -- amd-distributed/all2all/reference.py:10-17
* ``RankTestData``   -- amd-distributed/all2all/reference.py:21-51
* ``generate_input`` -- amd-distributed/all2all/reference.py:237-253
* ``input_t`` / ``output_t`` -- amd-distributed/all2all/task.py:8-9

Differences, all deliberate: inputs are drawn from a *CPU* generator seeded with
``seed + rank`` (the reference seeds a CUDA generator, which cannot be replayed
on a machine without a GPU) and then moved to the requested device, so the CPU
checker and the GPU path consume identical bytes; the dtype, the weight
distribution, the routing distribution and whether ``num_tokens`` is random are
parameters, because the benchmark workloads use bf16 / softmax weights / a fixed
token count whereas the reference task uses fp16 / uniform weights / a random
count.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

import torch


@dataclasses.dataclass
class MoEConfig:
    """Hyper-parameters of one all-to-all problem (reference.py:10-17)."""

    num_experts: int
    experts_per_token: int
    hidden_dim: int
    max_num_tokens: int
    in_dtype: torch.dtype = torch.bfloat16
    out_dtype: torch.dtype = torch.bfloat16


class RankTestData:
    """Inputs owned by one data-parallel rank (reference.py:21-51).

    ``indices [num_tokens, K] int32`` holds K distinct experts per token,
    ``weights [num_tokens, K] fp32`` the top-k weights and
    ``x [num_tokens, H]`` the token rows in ``cfg.in_dtype``.
    """

    def __init__(
        self,
        cfg: MoEConfig,
        rng: torch.Generator,
        rank: int,
        *,
        device: Optional[torch.device] = None,
        routing: str = "uniform",
        weights: str = "softmax",
        ragged: bool = False,
        zipf_s: float = 1.2,
    ):
        E, K, H, T = cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens
        if ragged:
            # reference.py:24-28 draws from [1, max_num_tokens); keep 1 when that range is empty
            self.num_tokens = int(torch.randint(1, T, [1], generator=rng).item()) if T > 1 else 1
        else:
            self.num_tokens = T
        n = self.num_tokens
        if routing == "uniform":
            # reference.py:33-35: a fresh permutation per token, first K entries
            idx = torch.empty(n, K, dtype=torch.int32)
            for i in range(n):
                idx[i] = torch.randperm(E, generator=rng)[:K]
        elif routing == "zipf":
            # expert popularity p_e ~ (e+1)^-s, sampled without replacement per token
            p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** zipf_s
            idx = torch.multinomial(p.expand(n, E), K, replacement=False, generator=rng).to(torch.int32)
        else:
            raise ValueError(f"unknown routing {routing!r}")
        if weights == "softmax":
            w = torch.softmax(torch.randn(n, K, generator=rng, dtype=torch.float32), dim=-1)
        elif weights == "rand":
            w = torch.rand(n, K, generator=rng, dtype=torch.float32)  # reference.py:37-43
        else:
            raise ValueError(f"unknown weights {weights!r}")
        x = torch.randn(n, H, generator=rng, dtype=torch.float32).to(cfg.in_dtype)
        dev = torch.device("cpu") if device is None else torch.device(device)
        self.indices = idx.to(dev)
        self.weights = w.to(dev)
        self.x = x.to(dev)

    def to(self, device) -> "RankTestData":
        """A copy of this rank's inputs on ``device`` (host or GPU)."""
        out = object.__new__(RankTestData)
        out.num_tokens = self.num_tokens
        out.indices = self.indices.to(device)
        out.weights = self.weights.to(device)
        out.x = self.x.to(device)
        return out


input_t = Tuple[MoEConfig, RankTestData, int, int]
output_t = torch.Tensor


def generate_input(
    num_experts: int,
    experts_per_token: int,
    hidden_dim: int,
    max_num_tokens: int,
    seed: int,
    rank: int,
    world_size: int,
    *,
    dtype: torch.dtype = torch.bfloat16,
    routing: str = "uniform",
    weights: str = "softmax",
    ragged: bool = False,
    device=None,
) -> input_t:
    """Build ``(cfg, rank_data, rank, world_size)`` for one rank (reference.py:237-253)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed + rank)
    cfg = MoEConfig(
        num_experts=num_experts,
        experts_per_token=experts_per_token,
        hidden_dim=hidden_dim,
        max_num_tokens=max_num_tokens,
        in_dtype=dtype,
        out_dtype=dtype,
    )
    rank_data = RankTestData(cfg, gen, rank, device=device, routing=routing, weights=weights, ragged=ragged)
    return cfg, rank_data, rank, world_size


# Benchmark workloads: shapes, routing and seeds of the five configurations the
# metric is quoted on.  "world" is the world size the configuration is defined
# for; c4 is also run at world sizes 1, 2 and 4 with experts split evenly.
WORKLOADS = {
    "c1": dict(num_experts=8, experts_per_token=2, hidden_dim=2048, max_num_tokens=16, seed=0, world=2),
    "c2": dict(num_experts=8, experts_per_token=2, hidden_dim=6144, max_num_tokens=128, seed=1, world=8),
    "c3": dict(num_experts=64, experts_per_token=6, hidden_dim=2048, max_num_tokens=256, seed=2, world=8,
               routing="zipf"),
    "c4": dict(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=256, seed=3, world=8),
    "c5": dict(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=256, seed=4, world=8,
               payload="fp8"),
}


def workload_input(name: str, rank: int, world_size: Optional[int] = None, device=None) -> input_t:
    """Inputs of benchmark workload ``name`` for ``rank`` (optionally at another world size)."""
    w = dict(WORKLOADS[name])
    ws = world_size if world_size is not None else w["world"]
    w.pop("world")
    w.pop("payload", None)
    return generate_input(rank=rank, world_size=ws, device=device, **w)


# The reference task's own test and benchmark shapes (amd-distributed/all2all/task.yml:48-65):
# (num_experts, experts_per_token, hidden_dim, max_num_tokens, seed), all at world size 8, fp16.
REFERENCE_TESTS = [
    (8, 2, 6144, 4, 1236), (64, 6, 2048, 4, 1234), (64, 6, 2048, 8, 542),
    (128, 4, 2880, 16, 347), (128, 4, 2880, 32, 51), (128, 8, 4096, 64, 175),
    (128, 8, 4096, 128, 534), (256, 8, 7168, 64, 897), (256, 8, 7168, 128, 4),
]
REFERENCE_BENCHMARKS = [
    (8, 2, 6144, 16, 6635), (64, 6, 2048, 32, 1234), (128, 4, 2880, 128, 51),
    (128, 8, 4096, 256, 175), (256, 8, 7168, 256, 4),
]


def reference_task_input(spec, rank: int, world_size: int = 8, device=None) -> input_t:
    """Inputs in the style of the reference task: fp16, uniform weights, random token count."""
    E, K, H, T, seed = spec
    return generate_input(E, K, H, T, seed, rank, world_size, dtype=torch.float16,
                          routing="uniform", weights="rand", ragged=True, device=device)
