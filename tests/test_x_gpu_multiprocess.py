"""The real deployment shape: one process per GPU, NCCL for the one handle all_gather,
CUDA IPC peer mappings, every rank running the fused call concurrently.  Needs >= 2 GPUs.

The parent computes the expected outputs ONCE with the CPU checker and hands every worker
only its own rank's inputs and expectation (files in a temporary directory), so the
workers spend their time on the GPU path, not on eight copies of the same CPU work."""
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

import gpu_mode_kernels_b200 as pkg
from oracle import a2a_oracle as O
from parity import quantised_inputs

pytestmark = pytest.mark.gpu

# (E, K, H, T, seed, back-to-back calls, payload, schedule, combine)
CASES = [
    (8, 2, 2048, 16, 0, 4, "direct", "phased", "pull"),
    (64, 6, 2048, 64, 2, 30, "direct", "phased", "pull"),
    (256, 8, 7168, 256, 3, 20, "direct", "phased", "pull"),
    # many items per block and strongly different token counts per rank: a combine block that got ahead
    # of this rank's own routing would read a stale slot
    (64, 6, 2048, 1024, 7, 12, "direct", "phased", "pull"),
    (256, 8, 7168, 256, 3, 20, "dedup", "phased", "pull"),
    (256, 8, 7168, 256, 4, 20, "fp8", "phased", "pull"),
    (64, 6, 2048, 64, 2, 30, "dedup", "pipelined", "push"),
    (256, 8, 7168, 256, 3, 20, "dedup", "pipelined", "push"),
    (256, 8, 7168, 256, 3, 20, "dedup", "pipelined", "pull"),
    (64, 6, 2048, 1024, 7, 12, "dedup", "pipelined", "push"),
    (256, 8, 7168, 256, 4, 20, "fp8", "pipelined", "push"),
]


def _prepare(ws, tmp):
    """Two alternating input sets per case; expectation per rank from the CPU checker."""
    for ci, (E, K, H, T, seed, _, payload, _, _) in enumerate(CASES):
        for si, sd in enumerate((seed, seed + 1000)):
            datas = [pkg.generate_input(E, K, H, T, seed=sd, rank=r, world_size=ws, ragged=True) for r in range(ws)]
            cfg = datas[0][0]
            rds = [d[1] for d in datas]
            _, ys = O.simulate(cfg, ws, rds)
            ys_q = O.simulate(cfg, ws, quantised_inputs(rds, cfg.in_dtype))[1] if payload == "fp8" else [None] * ws
            for r in range(ws):
                torch.save({"x": rds[r].x, "indices": rds[r].indices, "weights": rds[r].weights,
                            "num_tokens": rds[r].num_tokens, "y": ys[r], "y_q": ys_q[r]},
                           os.path.join(tmp, f"c{ci}_s{si}_r{r}.pt"))


def _within(got, want, tol):
    diff = (got.float() - want.float()).abs()
    return diff / (tol + tol * want.float().abs())


def _worker(rank, ws, port, tmp, q):
    import torch.distributed as dist

    from gpu_mode_kernels_b200.all2all import _CONTEXTS, custom_kernel

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.set_num_threads(2)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=torch.device(f"cuda:{rank}"))
    ok, msg = True, ""
    try:
        for ci, (E, K, H, T, seed, iters, payload, schedule, combine) in enumerate(CASES):
            cfg = pkg.MoEConfig(E, K, H, T)
            sets = []
            for si in range(2):
                d = torch.load(os.path.join(tmp, f"c{ci}_s{si}_r{rank}.pt"))
                rd = object.__new__(pkg.RankTestData)
                rd.num_tokens = d["num_tokens"]
                rd.x, rd.indices, rd.weights = (d[k].to(f"cuda:{rank}") for k in ("x", "indices", "weights"))
                sets.append((rd, d["y"], d["y_q"]))
            # like the task harness (my_eval.py:160-161) every rank is at the starting line before the
            # first launch: a rank still busy on the host would otherwise eat into the peers' wait budget
            torch.cuda.synchronize()
            dist.barrier()
            outs = []
            for i in range(iters):  # back to back, no host sync: epochs and slab reuse under real concurrency
                outs.append(custom_kernel((cfg, sets[i % 2][0], rank, ws), payload=payload, schedule=schedule,
                                          combine=combine))
            torch.cuda.synchronize()
            for ctx in _CONTEXTS.values():
                ctx.check()
            # alternating inputs: a flag that overtook its data would hand a consumer the other set's rows
            for i in range(2, iters):
                if not torch.equal(outs[i].view(torch.int16), outs[i - 2].view(torch.int16)):
                    ok, msg = False, f"case {ci} {payload}/{schedule}/{combine}: call {i} differs from call {i - 2}"
            for i in (0, 1):
                _, y, y_q = sets[i]
                got = outs[i].cpu()
                if payload == "fp8":
                    # every element within 2e-2 of the checker on the dequantised inputs; against the bf16
                    # reference at 6e-2 a 1e-4 fraction may reach 1.25x (e4m3's 1/17 worst case, see parity.py)
                    r1, r2 = _within(got, y_q, 2e-2), _within(got, y, 6e-2)
                    good = float(r1.max()) <= 1 and float(r2.max()) <= 1.25 and \
                        int((r2 > 1).sum()) <= max(1, int(1e-4 * r2.numel()))
                else:
                    good = float(_within(got, y, 2e-2).max()) <= 1
                if not good:
                    ok, msg = False, f"case {ci} {payload}/{schedule}/{combine}: output of call {i} outside tolerance"
            if not ok:
                break
            dist.barrier()
    except Exception as e:  # noqa: BLE001
        ok, msg = False, repr(e)
    q.put((rank, ok, msg))
    if ok:
        dist.destroy_process_group()  # hook releases the contexts (barrier first)
    else:
        q.close()
        q.join_thread()
        os._exit(1)  # no further collective after a failure: the peers may be somewhere else


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_custom_kernel_over_ipc(ws):
    if torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        _prepare(ws, tmp)
        procs = [ctx.Process(target=_worker, args=(r, ws, 29800 + ws, tmp, q), daemon=True) for r in range(ws)]
        for p in procs:
            p.start()
        res = [q.get(timeout=300) for _ in range(ws)]
        for p in procs:
            p.join(30)
    bad = [r for r in res if not r[1]]
    assert not bad, bad
