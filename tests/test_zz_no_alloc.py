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
