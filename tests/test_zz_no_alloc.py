"""a2a_route_noalloc: the routing entry point for callers that cannot allocate device memory.

Called through the C ABI and compared with the existing entry points (a2a_route +
a2a_copy_route) -- integer tables, so the comparison is exact -- on two calls in a row with
different inputs: the second call finds the first call's bits in the shared static array and
must not be disturbed by them.  The file is named to be collected last.
"""
import ctypes as C

import pytest
import torch

import gpu_mode_kernels_b200 as pkg
from gpu_mode_kernels_b200 import _lib
from gpu_mode_kernels_b200.all2all import A2AContext

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _route_noalloc(idx, E, K):
    lib = _lib.load()
    n = idx.shape[0]
    slots = torch.full((n, K), -7, dtype=torch.int32, device=DEV)   # outputs are the caller's
    counts = torch.full((E,), -7, dtype=torch.int32, device=DEV)
    rc = lib.a2a_route_noalloc(C.c_void_p(idx.data_ptr()), n, E, K, C.c_void_p(slots.data_ptr()),
                               C.c_void_p(counts.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, slots, counts


def test_no_alloc_routing_matches_context_routing_twice_in_a_row():
    torch.cuda.set_device(0)
    E, K, T = 256, 8, 256
    ctx = A2AContext(pkg.MoEConfig(E, K, 64, T), 0, 1, device=0)
    try:
        # first call: every token, a dense bitmap; second call: fewer tokens, other experts,
        # one out-of-range index and one repeated expert (both must come out as -1)
        g = torch.Generator().manual_seed(1)
        first = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
        second = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T // 3)]).to(torch.int32)
        second[5, 2] = E + 3
        second[9, 4] = second[9, 1]
        for idx_cpu in (first, second):
            idx = idx_cpu.to(DEV)
            ctx.route(idx)
            want_slots, want_counts = ctx.route_tables()
            rc, slots, counts = _route_noalloc(idx, E, K)
            assert rc == 0, _lib.strerror(rc)
            torch.cuda.synchronize()
            assert torch.equal(slots, want_slots)
            assert torch.equal(counts, want_counts)
            ctx.clear_status()
        assert slots[5, 2].item() == -1 and slots[9, 4].item() == -1
    finally:
        ctx.close()


def test_no_alloc_routing_at_its_limits_and_with_no_tokens():
    """The largest request the static tables take (4096 tokens, 1024 experts, top-32: several tokens
    per thread, 128 bitmap words per expert, the far end of the array in use) and an empty one, each
    after a smaller call that left its bits behind; checked against the CPU routing of the checker."""
    from oracle import a2a_oracle as O

    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(7)
    small = torch.stack([torch.randperm(64, generator=g)[:4] for _ in range(100)]).to(torch.int32)
    rc, _, _ = _route_noalloc(small.to(DEV), 64, 4)
    assert rc == 0
    E, K, T = 1024, 32, 4096
    big = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    rc, slots, counts = _route_noalloc(big.to(DEV), E, K)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    want_slots, want_counts = O.route_tables(big, E)
    assert torch.equal(slots.cpu(), want_slots) and torch.equal(counts.cpu(), want_counts)
    # no tokens at all, right after the dense call: every count is zero, nothing else is written
    empty = torch.zeros(0, 8, dtype=torch.int32, device=DEV)
    rc, slots, counts = _route_noalloc(empty, 256, 8)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert slots.numel() == 0 and torch.equal(counts.cpu(), torch.zeros(256, dtype=torch.int32))
    # and a normal call after that is undisturbed
    rc, slots, counts = _route_noalloc(small.to(DEV), 64, 4)
    torch.cuda.synchronize()
    want_slots, want_counts = O.route_tables(small, 64)
    assert rc == 0 and torch.equal(slots.cpu(), want_slots) and torch.equal(counts.cpu(), want_counts)


def test_no_alloc_routing_rejects_sizes_beyond_its_static_tables():
    torch.cuda.set_device(0)
    idx = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    lib = _lib.load()
    out = torch.zeros(4096, dtype=torch.int32, device=DEV)
    args = (C.c_void_p(out.data_ptr()), C.c_void_p(out.data_ptr()), None)
    assert lib.a2a_route_noalloc(C.c_void_p(idx.data_ptr()), 4097, 8, 2, *args) == _lib.A2A_ERR_CONFIG
    assert lib.a2a_route_noalloc(C.c_void_p(idx.data_ptr()), 4, 1025, 2, *args) == _lib.A2A_ERR_CONFIG
    assert lib.a2a_route_noalloc(C.c_void_p(idx.data_ptr()), 4, 8, 33, *args) == _lib.A2A_ERR_CONFIG
    assert "invalid" in _lib.strerror(_lib.A2A_ERR_CONFIG)
