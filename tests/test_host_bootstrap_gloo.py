"""The host-side bootstrap of a multi-rank context, two CPU ranks on gloo, against a fake of the
C library: one all_gather of the handle blobs, every peer opened from the gathered blobs in rank
order, a barrier before first use, contexts cached per configuration and released (after a barrier)
by the destroy_process_group hook."""
import ctypes as C
import os

import torch
import torch.multiprocessing as mp


class FakeLib:
    """Records what the host layer asks of liba2a.so; returns success."""

    def __init__(self, rank):
        self.rank, self.calls, self.opened = rank, [], None

    def a2a_create(self, handle_ref, cfg_ref):
        self.calls.append(("create", cfg_ref._obj.rank, cfg_ref._obj.world_size, cfg_ref._obj.payload))
        handle_ref._obj.value = 0x1000 + self.rank
        return 0

    def a2a_ipc_handle_bytes(self):
        return 64

    def a2a_export_handle(self, h, out):
        C.memset(out.value, 0xA0 + self.rank, 64)
        self.calls.append(("export",))
        return 0

    def a2a_open_peers(self, h, blobs):
        self.opened = bytes((C.c_ubyte * 128).from_address(blobs.value))
        self.calls.append(("open",))
        return 0

    def a2a_forward(self, h, x, idx, w, y, n, stream):
        self.calls.append(("forward", n))
        return 0

    def a2a_destroy(self, h):
        self.calls.append(("destroy",))
        return 0


def _worker(rank, port, q):
    import torch.distributed as dist

    from gpu_mode_kernels_b200 import _lib, all2all
    import gpu_mode_kernels_b200 as pkg

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    fake = FakeLib(rank)
    _lib.load = lambda: fake  # the host layer asks _lib for the library
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    ctx = all2all._context_for(cfg, rank, 2, 0, "dedup")
    again = all2all._context_for(cfg, rank, 2, 0, "dedup")
    other = all2all._context_for(cfg, rank, 2, 0, "direct")
    ok = again is ctx and other is not ctx
    ok = ok and fake.opened == bytes([0xA0] * 64 + [0xA1] * 64)  # both blobs, rank order
    ok = ok and [c[0] for c in fake.calls[:3]] == ["create", "export", "open"]
    ok = ok and fake.calls[0] == ("create", rank, 2, _lib.PAYLOAD["dedup"])
    dist.destroy_process_group()  # the hook releases both cached contexts first
    ok = ok and [c[0] for c in fake.calls].count("destroy") == 2 and not all2all._CONTEXTS
    q.put((rank, bool(ok), fake.calls))


def test_two_rank_bootstrap_and_release_on_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 29731, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(60)
    assert all(r[1] for r in res), res
