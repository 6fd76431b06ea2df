"""The host side of a multi-rank context, CPU ranks on gloo, against a fake of the device
part of the C library (creation, IPC, launches) -- the configuration fingerprint and the check
of the gathered handle blobs are the REAL library's, which need no device:

* bootstrap: one all_gather of the handle blobs, peers opened from the gathered blobs in rank
  order, a barrier before first use, contexts cached per configuration and released (after a
  barrier) by the destroy_process_group hook;
* a rank created with another payload is refused at set-up on every rank, with a message
  naming the rank that differs; so is a truncated gather;
* a rank that leaves between two steps: the survivor's next call ends in A2A_ERR_TIMEOUT (the
  device's bounded wait, simulated by the fake's status word), the call after that raises it,
  clears it, and the context is usable again.  No GPU is involved anywhere."""
import ctypes as C
import os

import torch
import torch.multiprocessing as mp


class FakeLib:
    """Records what the host layer asks of liba2a.so.  Device work is faked; fingerprints and the
    blob check are delegated to the real library."""

    def __init__(self, rank, real):
        self.rank, self.real, self.calls, self.opened = rank, real, [], None
        self.cfg = None
        self.status_code = 0      # what the device-side status word would hold
        self.peer_gone = False    # the next forward waits for a peer that has left
        self.msg = C.create_string_buffer(200)

    def a2a_create(self, handle_ref, cfg_ref):
        self.cfg = cfg_ref._obj
        self.calls.append(("create", self.cfg.rank, self.cfg.world_size, self.cfg.payload, self.cfg.schedule,
                           self.cfg.chunks))
        handle_ref._obj.value = 0x1000 + self.rank
        return 0

    def a2a_ipc_handle_bytes(self):
        return self.real.a2a_ipc_handle_bytes()

    def a2a_export_handle(self, h, out):
        C.memset(out.value, 0xA0 + self.rank, 64)  # stands for the CUDA IPC handle
        rc = self.real.a2a_fingerprint(C.byref(self.cfg), C.c_void_p(out.value + 64))
        self.calls.append(("export",))
        return rc

    def a2a_open_peers(self, h, blobs, nbytes):
        self.opened = bytes((C.c_ubyte * nbytes).from_address(blobs.value))
        self.calls.append(("open",))
        return self.real.a2a_check_handles(C.byref(self.cfg), blobs, nbytes, self.msg, 200)

    def a2a_last_error(self, h):
        return self.msg.value

    def a2a_status_peek(self, h):
        return self.status_code

    def a2a_status(self, h, out_ref):
        out_ref._obj.code, out_ref._obj.rank, out_ref._obj.peer, out_ref._obj.phase = self.status_code, self.rank, 1, 3
        return 0

    def a2a_status_clear(self, h):
        self.calls.append(("clear",))
        self.status_code = 0
        return 0

    def a2a_forward_host(self, h, x, idx, w, y, n, stream):
        self.calls.append(("forward_host", n))
        if self.peer_gone:  # the kernel's bounded wait would run out and record this
            self.status_code = 3
        return 0

    def a2a_destroy(self, h):
        self.calls.append(("destroy",))
        return 0

    def a2a_strerror(self, code):
        return self.real.a2a_strerror(code)


class _FakeStream:
    cuda_stream = 0

    def synchronize(self):
        pass


def _setup(rank, ws, port):
    import torch.distributed as dist

    from gpu_mode_kernels_b200 import _lib, all2all

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    fake = FakeLib(rank, _lib.load())
    _lib.load = lambda: fake  # the host layer asks _lib for the library
    torch.cuda.current_device = lambda: 0
    torch.cuda.current_stream = lambda *a, **k: _FakeStream()
    return dist, _lib, all2all, fake


def _bootstrap_worker(rank, port, q):
    import gpu_mode_kernels_b200 as pkg

    dist, _lib, all2all, fake = _setup(rank, 2, port)
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    os.environ["A2A_CHUNKS"] = "2"  # resolved on the host and carried in the configuration
    ctx = all2all._context_for(cfg, rank, 2, 0, "dedup", "phased", "pull")
    again = all2all._context_for(cfg, rank, 2, 0, "dedup", "phased", "pull")
    other = all2all._context_for(cfg, rank, 2, 0, "direct", "auto", "push")  # DIRECT has no pipelined form
    piped = all2all._context_for(cfg, rank, 2, 0, "dedup", "auto", "push")
    ok = again is ctx and other is not ctx and piped is not ctx
    ok = ok and fake.opened[:64] == bytes([0xA0] * 64) and fake.opened[128:192] == bytes([0xA1] * 64)  # rank order
    ok = ok and [c[0] for c in fake.calls[:3]] == ["create", "export", "open"]
    ok = ok and fake.calls[0] == ("create", rank, 2, _lib.PAYLOAD["dedup"], _lib.SCHEDULE["phased"], 2)
    creates = [c for c in fake.calls if c[0] == "create"]
    ok = ok and creates[1][3:5] == (_lib.PAYLOAD["direct"], _lib.SCHEDULE["phased"])
    ok = ok and creates[2][3:6] == (_lib.PAYLOAD["dedup"], _lib.SCHEDULE["pipelined"], 1)
    dist.destroy_process_group()  # the hook releases the cached contexts first
    ok = ok and [c[0] for c in fake.calls].count("destroy") == 3 and not all2all._CONTEXTS
    q.put((rank, bool(ok), fake.calls))


def _mismatch_worker(rank, port, q):
    import gpu_mode_kernels_b200 as pkg

    dist, _lib, all2all, fake = _setup(rank, 2, port)
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    msgs = []
    # (a) rank 1 asks for another payload than rank 0: both refuse, naming the rank that differs from them
    try:
        all2all.A2AContext(cfg, rank, 2, device=0, payload="dedup" if rank == 0 else "direct")
        msgs.append("no error")
    except _lib.A2AError as e:
        msgs.append((e.code, str(e)))
    # (b) another chunk count on rank 1 (what two ranks with different A2A_CHUNKS used to do silently)
    try:
        all2all.A2AContext(pkg.MoEConfig(8, 2, 64, 128), rank, 2, device=0, payload="dedup", chunks=1 + rank)
        msgs.append("no error")
    except _lib.A2AError as e:
        msgs.append((e.code, str(e)))
    # (c) a gather that came back short
    ctx = all2all.A2AContext(cfg, rank, 2, device=0, payload="dedup", connect=False)
    blob = ctx.export_handle()
    try:
        ctx.open_peers(torch.cat([blob, blob])[:-7])
        msgs.append("no error")
    except _lib.A2AError as e:
        msgs.append((e.code, str(e)))
    # (d) a damaged blob
    bad = torch.cat([blob, blob]).clone()
    bad[64 + 128 * (1 - rank)] ^= 0xFF
    try:
        ctx.open_peers(bad)
        msgs.append("no error")
    except _lib.A2AError as e:
        msgs.append((e.code, str(e)))
    # (e) and the good case still passes
    ctx.open_peers(torch.cat([blob, blob]))
    other = 1 - rank
    ok = (msgs[0][0] == 1 and f"rank {other} was created with a different configuration" in msgs[0][1]
          and msgs[1][0] == 1 and f"rank {other}" in msgs[1][1]
          and msgs[2][0] == 1 and "bytes" in msgs[2][1]
          and msgs[3][0] == 1 and "damaged" in msgs[3][1])
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, bool(ok), msgs))


def _leaver_worker(rank, port, q):
    import gpu_mode_kernels_b200 as pkg

    dist, _lib, all2all, fake = _setup(rank, 2, port)
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    _, rd, _, _ = pkg.generate_input(8, 2, 64, 4, seed=1, rank=rank, world_size=2)
    data = (cfg, rd, rank, 2)
    all2all.custom_kernel(data)  # step 1: both ranks
    dist.barrier()
    log = []
    if rank == 1:
        # leaves between steps: nothing of it is in flight; it tells nobody
        q.put((rank, True, "left"))
        return
    fake.peer_gone = True
    all2all.custom_kernel(data)  # step 2: returns (the wait on the device is bounded), status = TIMEOUT
    log.append(fake.status_code)
    try:
        all2all.custom_kernel(data)  # step 3: the recorded timeout is raised before anything is launched
        log.append("no error")
    except _lib.A2AError as e:
        log.append((e.code, "peer 1" in str(e)))
    log.append([c[0] for c in fake.calls].count("forward_host"))  # still 2: step 3 launched nothing
    log.append(fake.status_code)                                   # cleared by the raise
    fake.peer_gone = False
    all2all.custom_kernel(data)  # the context is usable again
    log.append([c[0] for c in fake.calls].count("forward_host"))
    ok = log == [3, (3, True), 2, 0, 3] and ("clear",) in fake.calls
    all2all.release_contexts(barrier=False)  # no collective with a rank that has left
    q.put((rank, bool(ok), log))


def _run(worker, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(60)
    assert all(r[1] for r in res), res


def test_two_rank_bootstrap_and_release_on_gloo():
    _run(_bootstrap_worker, 29731)


def test_ranks_that_disagree_are_refused_at_setup():
    _run(_mismatch_worker, 29732)


def test_rank_that_leaves_between_steps_gives_a_timeout_then_a_usable_context():
    _run(_leaver_worker, 29733)
