"""Several ranks on ONE GPU, run phase by phase in one process.

Kernels that wait on a peer must never share a GPU with the kernel they wait
for, so the ranks here are stepped in lock-step: every rank's sending kernel is
enqueued before any rank's waiting kernel, on one stream, and each wait finds its
flag already set.  The kernels, addresses, flags and epochs are exactly those of
a real multi-GPU run; only CUDA IPC and true concurrency are not exercised.
Validation tool: parity tests and the smoke check use it to cover world sizes
2, 4 and 8 on a single device.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .all2all import A2AContext
from .task import MoEConfig


class LocalWorld:
    def __init__(self, cfg: MoEConfig, world_size: int, *, payload: str = "direct", schedule: str = "phased",
                 combine: str = "pull", timeout_ms: int = 2000, device: int = 0):
        self.cfg, self.world_size = cfg, world_size
        self.ctxs: List[A2AContext] = [
            A2AContext(cfg, r, world_size, device=device, payload=payload, schedule=schedule, combine=combine,
                       timeout_ms=timeout_ms, connect=False)
            for r in range(world_size)
        ]
        A2AContext.attach_local(self.ctxs)

    def dispatch(self, rank_datas: Sequence) -> None:
        """route + dispatch on every rank (rank_datas hold device tensors)."""
        for c, rd in zip(self.ctxs, rank_datas):
            c.route(rd.indices)
        for c, rd in zip(self.ctxs, rank_datas):
            c.dispatch_send(rd.x)
        for c in self.ctxs:
            c.dispatch_recv()

    def forward_phases(self, rank_datas: Sequence) -> List[torch.Tensor]:
        """The four public phases, one after the other."""
        self.dispatch(rank_datas)
        for c in self.ctxs:
            c.expert_placeholder()
        return [c.combine(rd.weights) for c, rd in zip(self.ctxs, rank_datas)]

    def forward(self, rank_datas: Sequence) -> List[torch.Tensor]:
        """The kernels a2a_forward launches (route, send, recv+expert fused, combine), in lock-step."""
        for c, rd in zip(self.ctxs, rank_datas):
            c.route(rd.indices)
        for c, rd in zip(self.ctxs, rank_datas):
            c.dispatch_send(rd.x)
        for c in self.ctxs:
            c.dispatch_recv_expert()
        return [c.combine(rd.weights) for c, rd in zip(self.ctxs, rank_datas)]

    def forward_pipelined(self, rank_datas: Sequence) -> List[torch.Tensor]:
        """The roles of the pipelined one-launch kernel as three launches per rank, in lock-step:
        every rank's senders and routers, then every rank's expert blocks, then every rank's combine."""
        for c, rd in zip(self.ctxs, rank_datas):
            c.pipe_step(0, rd.x, rd.indices, rd.weights)
        for c in self.ctxs:
            c.pipe_step(1)
        return [c.pipe_step(2) for c in self.ctxs]

    def check(self) -> None:
        for c in self.ctxs:
            c.check()

    def close(self) -> None:
        torch.cuda.synchronize()
        for c in self.ctxs:
            c.close()
