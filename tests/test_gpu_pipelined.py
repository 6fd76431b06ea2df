"""GPU parity of the pipelined schedule (role-specialised one-launch kernel), both combine modes.

World sizes above one are stepped role by role on a single GPU (``LocalWorld.forward_pipelined``:
the same device code as the one-launch kernel, launched as senders+routers / experts / combine so
that a kernel that waits never shares the GPU with the kernel it waits for).  At world size one
the real one-launch kernel runs and must give the same bits as the stepped roles.  The
one-process-per-GPU form is covered by test_x_gpu_multiprocess.py.
"""
import pytest
import torch

import gpu_mode_kernels_b200 as pkg
from gpu_mode_kernels_b200 import _lib
from gpu_mode_kernels_b200.all2all import A2AContext, A2AError, custom_kernel, release_contexts
from gpu_mode_kernels_b200.local_world import LocalWorld
from oracle import a2a_oracle as O
from parity import check_y, fp8_roundtrip, tol

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
COMBINES = ["push", "pull"]


def bits(t):
    return t.contiguous().view(torch.int16)


def check_pipelined_dispatch(world, disp, dtype, payload="dedup"):
    """After a pipelined forward the slabs hold the expert OUTPUT of every dispatched row:
    counts and (expert, source, token, k) must equal the reference's dispatch exactly, and every row
    must be bit-equal to dtype(float(reference row) * (1 + rank)) -- one rounding, as reference.py:262."""
    for r, c in enumerate(world.ctxs):
        counts, rows, meta = c.export_dispatch()
        torch.cuda.synchronize()
        d = disp[r]
        assert torch.equal(counts.cpu(), d.expert_num_tokens), f"rank {r}: expert_num_tokens differ"
        n = counts.cpu().tolist()
        gmeta = torch.cat([meta[e, : n[e]] for e in range(len(n))], 0).cpu()
        grows = torch.cat([rows[e, : n[e]] for e in range(len(n))], 0).cpu()
        assert torch.equal(gmeta, d.meta), f"rank {r}: meta/order differ"
        rows_in = fp8_roundtrip(d.rows, dtype) if payload == "fp8" and d.rows.numel() else d.rows
        want = (rows_in.float() * float(1 + r)).to(dtype)
        assert torch.equal(bits(grows), bits(want)), f"rank {r}: rows differ"


def run_case(cfg, ws, rds_cpu, combine, tolerance=None, payload="dedup"):
    disp, ys = O.simulate(cfg, ws, rds_cpu)
    world = LocalWorld(cfg, ws, payload=payload, schedule="pipelined", combine=combine)
    try:
        rds = [rd.to(DEV) for rd in rds_cpu]
        out = world.forward_pipelined(rds)
        torch.cuda.synchronize()
        world.check()
        check_pipelined_dispatch(world, disp, cfg.in_dtype, payload)
        for r in range(ws):
            assert out[r].shape == (rds_cpu[r].num_tokens, cfg.hidden_dim) and out[r].dtype == cfg.out_dtype
        if payload == "fp8":
            check_y(cfg, ws, rds_cpu, out, ys, payload)  # the FP8 rules of parity.py
        else:
            t = tolerance or tol(cfg.in_dtype)
            for r in range(ws):
                torch.testing.assert_close(out[r].cpu().float(), ys[r].float(), **t)
        return world, out
    except Exception:
        world.close()
        raise


@pytest.mark.parametrize("combine", COMBINES)
def test_golden_cases(golden, combine):
    """Every golden case recorded from the reference."""
    ws = golden.ws
    rds_cpu = [golden.rank_data(r) for r in range(ws)]
    world, out = run_case(golden.cfg, ws, rds_cpu, combine)
    try:
        for r in range(ws):
            torch.testing.assert_close(out[r].cpu().float(), golden.expected_y(r).float(), **tol(golden.cfg.in_dtype))
    finally:
        world.close()


@pytest.mark.parametrize("combine", COMBINES)
@pytest.mark.parametrize("name,ws", [("c1", 2), ("c2", 8), ("c3", 8), ("c4", 8), ("c4", 4), ("c4", 2), ("c4", 1)])
def test_benchmark_workloads_full_size(name, ws, combine):
    """The benchmark configurations at full size; then a second call with other, ragged inputs on the
    same contexts (epochs advance, nothing stale survives)."""
    datas = [pkg.workload_input(name, r, ws) for r in range(ws)]
    cfg = datas[0][0]
    world, _ = run_case(cfg, ws, [d[1] for d in datas], combine)
    try:
        datas2 = [pkg.generate_input(cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens,
                                     seed=99, rank=r, world_size=ws, ragged=True) for r in range(ws)]
        rds2 = [d[1] for d in datas2]
        disp2, ys2 = O.simulate(cfg, ws, rds2)
        out2 = world.forward_pipelined([rd.to(DEV) for rd in rds2])
        torch.cuda.synchronize()
        world.check()
        check_pipelined_dispatch(world, disp2, cfg.in_dtype)
        for r in range(ws):
            torch.testing.assert_close(out2[r].cpu().float(), ys2[r].float(), **tol(cfg.in_dtype))
    finally:
        world.close()


@pytest.mark.parametrize("E,K,H,T,ws,dtype", [
    (8, 1, 8, 1, 8, torch.bfloat16),         # one token, one expert per rank, smallest row
    (4, 4, 2880, 3, 2, torch.float16),       # every expert chosen, row not a multiple of 2 KB
    (16, 2, 64, 1, 4, torch.bfloat16),       # single token per rank
    (1024, 32, 128, 40, 8, torch.bfloat16),  # limits of E and K
    (6, 3, 520, 33, 1, torch.float16),       # single rank, odd sizes
    (16, 4, 9216, 70, 2, torch.bfloat16),    # a row larger than one 16 KB stage of the senders' ring
    (32, 4, 256, 700, 4, torch.bfloat16),    # several rounds of 256 tokens in the list compaction
])
@pytest.mark.parametrize("combine", COMBINES)
def test_edge_shapes(E, K, H, T, ws, dtype, combine):
    datas = [pkg.generate_input(E, K, H, T, seed=5, rank=r, world_size=ws, dtype=dtype, ragged=(T > 2))
             for r in range(ws)]
    world, _ = run_case(datas[0][0], ws, [d[1] for d in datas], combine)
    world.close()


@pytest.mark.parametrize("combine", COMBINES)
@pytest.mark.parametrize("name,ws", [("c5", 8), ("c5", 2), ("c5", 1), ("c3", 8)])
def test_fp8_payload(name, ws, combine):
    """Config 5: the senders quantise each wire row to e4m3 + one fp32 scale per 128 values on the fly;
    the expert rank dequantises.  Dispatch bit-exact against the checker's quantise -> dequantise of
    the reference rows; combine under the FP8 rules (parity.py)."""
    datas = [pkg.workload_input(name, r, ws) for r in range(ws)]
    world, _ = run_case(datas[0][0], ws, [d[1] for d in datas], combine, payload="fp8")
    world.close()


@pytest.mark.parametrize("combine", COMBINES)
def test_fp8_edge_shapes(combine):
    for E, K, H, T, ws, dtype in [(8, 2, 128, 5, 2, torch.bfloat16), (16, 4, 2944, 70, 4, torch.float16),
                                  (32, 4, 256, 700, 4, torch.bfloat16), (6, 3, 640, 33, 1, torch.float16)]:
        datas = [pkg.generate_input(E, K, H, T, seed=6, rank=r, world_size=ws, dtype=dtype, ragged=True)
                 for r in range(ws)]
        world, _ = run_case(datas[0][0], ws, [d[1] for d in datas], combine, payload="fp8")
        world.close()


@pytest.mark.parametrize("combine", COMBINES)
def test_a_rank_without_tokens(combine):
    """One rank of three brings no tokens at all to a call (its experts still serve the others)."""
    ws, E, K, H, T = 3, 12, 3, 256, 40
    datas = [pkg.generate_input(E, K, H, T, seed=8, rank=r, world_size=ws, ragged=True) for r in range(ws)]
    cfg = datas[0][0]
    rds = [d[1] for d in datas]
    rds[1].num_tokens = 0
    rds[1].x, rds[1].indices, rds[1].weights = rds[1].x[:0], rds[1].indices[:0], rds[1].weights[:0]
    world, out = run_case(cfg, ws, rds, combine)
    try:
        assert out[1].shape == (0, H)
    finally:
        world.close()


@pytest.mark.parametrize("spec", pkg.REFERENCE_TESTS + pkg.REFERENCE_BENCHMARKS,
                         ids=lambda s: "E{}_K{}_H{}_T{}".format(*s[:4]))
def test_reference_task_shapes_fp16(spec):
    """The reference task's own shapes in its own style (fp16, uniform weights, random token counts)
    under its own tolerance rtol=1e-2, atol=5e-3 (reference.py:279), expert-side reduction on."""
    ws = 8
    datas = [pkg.reference_task_input(spec, r, ws) for r in range(ws)]
    world, _ = run_case(datas[0][0], ws, [d[1] for d in datas], "push", dict(rtol=1e-2, atol=5e-3))
    world.close()


@pytest.mark.parametrize("combine", COMBINES)
def test_one_launch_equals_stepped_roles_single_rank(combine):
    """World size 1 (no peer to wait for): the cooperative one-launch kernel gives the bits of the
    three stepped launches, and both match the checker."""
    cfg, rd, _, _ = pkg.workload_input("c2", 0, 1)
    _, ys = O.simulate(cfg, 1, [rd])
    ctx = A2AContext(cfg, 0, 1, device=0, payload="dedup", schedule="pipelined", combine=combine)
    world = LocalWorld(cfg, 1, payload="dedup", schedule="pipelined", combine=combine)
    try:
        d = rd.to(DEV)
        l0 = ctx.launches
        y = ctx.forward(d.x, d.indices, d.weights)
        assert ctx.launches - l0 == 1
        torch.cuda.synchronize()
        ctx.check()
        torch.testing.assert_close(y.cpu().float(), ys[0].float(), **tol(cfg.in_dtype))
        ref = world.forward_pipelined([d])[0]
        torch.cuda.synchronize()
        world.check()
        assert torch.equal(bits(ref), bits(y))
    finally:
        ctx.close()
        world.close()


@pytest.mark.parametrize("combine", COMBINES)
def test_repeated_calls_without_host_sync(combine):
    """Fifty back-to-back calls on one stream, inputs alternating: the last results are right."""
    ws = 4
    cfg = pkg.MoEConfig(32, 4, 512, 64)
    sets = []
    for seed in (1, 2):
        datas = [pkg.generate_input(32, 4, 512, 64, seed=seed, rank=r, world_size=ws, ragged=True) for r in range(ws)]
        _, ys = O.simulate(cfg, ws, [d[1] for d in datas])
        sets.append(([d[1].to(DEV) for d in datas], ys))
    world = LocalWorld(cfg, ws, payload="dedup", schedule="pipelined", combine=combine)
    try:
        outs = None
        for i in range(50):
            outs = world.forward_pipelined(sets[i % 2][0])
        torch.cuda.synchronize()
        world.check()
        for r in range(ws):
            torch.testing.assert_close(outs[r].cpu().float(), sets[1][1][r].float(), **tol(torch.bfloat16))
    finally:
        world.close()


@pytest.mark.parametrize("combine", COMBINES)
def test_bad_and_repeated_expert_indices_are_reported_and_dropped(combine):
    cfg = pkg.MoEConfig(8, 3, 64, 4)
    ctx = A2AContext(cfg, 0, 1, device=0, payload="dedup", schedule="pipelined", combine=combine)
    try:
        idx = torch.tensor([[0, 1, 2], [2, 9, 3], [4, 4, 5], [-1, 6, 7]], dtype=torch.int32, device=DEV)
        x = torch.ones(4, 64, dtype=torch.bfloat16, device=DEV)
        w = torch.tensor([[0.25, 0.25, 0.5], [0.5, 0.25, 0.25], [0.25, 0.5, 0.125], [0.5, 0.25, 0.25]], device=DEV)
        y = ctx.forward(x, idx, w)
        torch.cuda.synchronize()
        s = ctx.status()
        assert s.code == _lib.A2A_ERR_ROUTING and s.phase == 1 and s.rank == 0 and s.detail in (9, -1, 4)
        assert ctx.peek() == _lib.A2A_ERR_ROUTING
        # valid pairs still went through (scale 1 at rank 0)
        assert torch.equal(y[0].float().cpu(), torch.ones(64))
        assert torch.equal(y[1].float().cpu(), torch.full((64,), 0.75))   # the out-of-range pair dropped
        assert torch.equal(y[2].float().cpu(), torch.full((64,), 0.375))  # the repeated expert dropped
        assert torch.equal(y[3].float().cpu(), torch.full((64,), 0.5))
        slots, _ = ctx.route_tables()
        torch.cuda.synchronize()
        assert slots.cpu().tolist() == [[0, 0, 0], [1, -1, 0], [0, -1, 0], [-1, 0, 0]]
        ctx.clear_status()
        assert ctx.peek() == 0
        idx_ok = torch.tensor([[0, 1, 2], [2, 7, 3], [4, 6, 5], [1, 6, 7]], dtype=torch.int32, device=DEV)
        y = ctx.forward(x, idx_ok, w)
        torch.cuda.synchronize()
        ctx.check()
        assert torch.equal(y[0].float().cpu(), torch.ones(64))
    finally:
        ctx.close()


@pytest.mark.parametrize("schedule,combine", [("pipelined", "push"), ("pipelined", "pull"), ("phased", "pull")])
def test_absent_peer_times_out_and_the_same_contexts_work_again(schedule, combine):
    """A flag nothing sets: the bounded wait gives up, the status names the missing peer, the kernel
    returns normally.  After a2a_status_clear the SAME contexts run a correct forward."""
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    world = LocalWorld(cfg, 2, payload="dedup", schedule=schedule, combine=combine, timeout_ms=50)
    try:
        datas = [pkg.generate_input(8, 2, 64, 4, seed=1, rank=r, world_size=2) for r in range(2)]
        rds = [d[1].to(DEV) for d in datas]
        _, ys = O.simulate(cfg, 2, [d[1] for d in datas])
        c0 = world.ctxs[0]
        if schedule == "pipelined":
            c0.pipe_step(0, rds[0].x, rds[0].indices, rds[0].weights)
            c0.pipe_step(1)  # rank 1 never sends in this call
        else:
            c0.route(rds[0].indices)
            c0.dispatch_send(rds[0].x)
            c0.dispatch_recv()
        torch.cuda.synchronize()
        s = c0.status()
        assert s.code == _lib.A2A_ERR_TIMEOUT and s.peer == 1 and s.phase == 3 and s.rank == 0
        assert c0.peek() == _lib.A2A_ERR_TIMEOUT
        with pytest.raises(A2AError):
            c0.check()
        # while the timeout stands every wait gives up at once; clearing makes the context whole again
        for c in world.ctxs:
            c.clear_status()
        # rank 1 missed one call: bring its call counter level with rank 0's (a call of its own that
        # waits for nobody: it only sends)
        c1 = world.ctxs[1]
        if schedule == "pipelined":
            c1.pipe_step(0, rds[1].x, rds[1].indices, rds[1].weights)
        else:
            c1.route(rds[1].indices)
            c1.dispatch_send(rds[1].x)
        out = world.forward_pipelined(rds) if schedule == "pipelined" else world.forward(rds)
        torch.cuda.synchronize()
        world.check()
        for r in range(2):
            torch.testing.assert_close(out[r].cpu().float(), ys[r].float(), **tol(torch.bfloat16))
    finally:
        world.close()


def test_custom_kernel_raises_at_the_next_call_and_recovers():
    """The plugin entry looks at the status before every call: an error recorded by the previous
    call is raised (and cleared), the call after that runs normally."""
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    _, rd, _, _ = pkg.generate_input(8, 2, 64, 4, seed=3, rank=0, world_size=1, device=DEV)
    _, ys = O.simulate(cfg, 1, [rd.to("cpu")])
    try:
        bad = object.__new__(pkg.RankTestData)
        bad.num_tokens, bad.x, bad.weights = rd.num_tokens, rd.x, rd.weights
        bad.indices = rd.indices.clone()
        bad.indices[1, 1] = 99
        custom_kernel((cfg, bad, 0, 1))  # records A2A_ERR_ROUTING; the call itself returns
        torch.cuda.synchronize()
        with pytest.raises(A2AError) as ei:
            custom_kernel((cfg, rd, 0, 1))
        assert ei.value.code == _lib.A2A_ERR_ROUTING
        y = custom_kernel((cfg, rd, 0, 1))
        torch.cuda.synchronize()
        torch.testing.assert_close(y.cpu().float(), ys[0].float(), **tol(cfg.in_dtype))
    finally:
        release_contexts(barrier=False)


def test_forward_refuses_tensors_it_would_misread():
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    ctx = A2AContext(cfg, 0, 1, device=0, payload="dedup", schedule="pipelined", combine="push")
    try:
        x = torch.ones(4, 64, dtype=torch.bfloat16, device=DEV)
        idx = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
        w = torch.ones(4, 2, device=DEV)
        for args in ((x, idx.long(), w), (x, idx, w.double()), (x.half(), idx, w), (x, idx, w[:, :1]),
                     (x.t().contiguous().t(), idx, w), (x.cpu(), idx, w)):
            with pytest.raises(A2AError) as ei:
                ctx.forward(*args)
            assert ei.value.code == _lib.A2A_ERR_CONFIG
        with pytest.raises(A2AError):
            ctx.forward_host(x, idx.cpu(), w.cpu())
    finally:
        ctx.close()


def test_pipelined_needs_a_wire_row_payload_and_push_needs_pipelined():
    cfg = pkg.MoEConfig(8, 2, 64, 4)
    for kw in (dict(payload="direct", schedule="pipelined"), dict(payload="dedup", schedule="phased", combine="push")):
        with pytest.raises(A2AError) as ei:
            A2AContext(cfg, 0, 1, device=0, **kw)
        assert ei.value.code == _lib.A2A_ERR_CONFIG
