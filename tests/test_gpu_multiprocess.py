"""The real deployment shape: one process per GPU, NCCL for the one handle all_gather,
CUDA IPC peer mappings, every rank running the fused call concurrently.  Needs >= 2 GPUs."""
import os

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, ws, port, cases, q):
    import torch.distributed as dist

    import gpu_mode_kernels_b200 as pkg
    from gpu_mode_kernels_b200.all2all import custom_kernel, _CONTEXTS
    from oracle import a2a_oracle as O
    from parity import check_y

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=torch.device(f"cuda:{rank}"))
    ok, msg = True, ""
    try:
        for (E, K, H, T, seed, iters, payload) in cases:
            # two different input sets, alternated: a flag that overtook its data would hand a
            # consumer the other set's rows, which the comparison catches
            sets = []
            for sd in (seed, seed + 1000):
                datas = [pkg.generate_input(E, K, H, T, seed=sd, rank=r, world_size=ws, ragged=True) for r in range(ws)]
                cfg = datas[0][0]
                rds_cpu = [d[1] for d in datas]
                _, ys = O.simulate(cfg, ws, rds_cpu)
                sets.append((rds_cpu, ys, datas[rank][1].to(f"cuda:{rank}")))
            outs = []
            for i in range(iters):  # back-to-back, no host sync: epochs and slab reuse under real concurrency
                outs.append(custom_kernel((cfg, sets[i % 2][2], rank, ws), payload=payload))
            torch.cuda.synchronize()
            for ctx in _CONTEXTS.values():
                ctx.check()
            try:
                for i in (0, 1, iters - 2, iters - 1):
                    rds_cpu, ys, _ = sets[i % 2]
                    check_y(cfg, ws, rds_cpu, {rank: outs[i]}, ys, payload, ranks=[rank])
                for i in range(2, iters):
                    assert torch.equal(outs[i].view(torch.int16), outs[i - 2].view(torch.int16)), f"iteration {i} differs"
            except AssertionError as e:  # noqa: PERF203
                ok, msg = False, f"case {(E, K, H, T, payload)}: {e}"
                break
            dist.barrier()
    except Exception as e:  # noqa: BLE001
        ok, msg = False, repr(e)
    finally:
        q.put((rank, ok, msg))
        dist.destroy_process_group()  # hook releases the contexts (barrier first)


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_custom_kernel_over_ipc(ws):
    if torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    cases = [(8, 2, 2048, 16, 0, 3, "direct"), (64, 6, 2048, 64, 2, 30, "direct"), (256, 8, 7168, 256, 3, 20, "direct"),
             (64, 6, 2048, 64, 2, 30, "dedup"), (256, 8, 7168, 256, 3, 20, "dedup"), (256, 8, 7168, 256, 4, 20, "fp8")]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, ws, 29800 + ws, cases, q)) for r in range(ws)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(ws)]
    for p in procs:
        p.join(60)
    bad = [r for r in res if not r[1]]
    assert not bad, bad
