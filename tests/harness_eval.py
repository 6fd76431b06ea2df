"""Stand-in for the reference task's evaluation harness (amd-distributed/all2all/my_eval.py).

    python tests/harness_eval.py test      [--world N]
    python tests/harness_eval.py benchmark [--world N]

Same structure and output format as the reference's harness: one process per GPU, a fresh
NCCL process group per case (my_eval.py:64-85), `custom_kernel(data)` checked against the
reference algorithm with the task's own tolerance rtol=1e-2 / atol=5e-3 (reference.py:275-283),
"test.N.status pass|fail" lines (my_eval.py:105-116); in benchmark mode the L2 is cleared, ranks
barrier, rank 0 takes wall-clock time around the call (my_eval.py:159-177) and
"benchmark.N.<runs|mean|std|err|best|worst>" lines in nanoseconds are printed (my_eval.py:272-280).
Differences: the shapes come from task.py's copy of task.yml's list, the inputs from this
repository's CPU generator in the task's style (fp16, uniform weights, random token count), and
the expectation handed to the package's `check_implementation` comes from the literal port of the
reference path in oracle/ run on the GPUs over NCCL, because the reference checkout is not on the
GPU machine.  Test infrastructure: lives under tests/.
"""
import argparse
import math
import os
import sys
import time

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _stats(durations):
    runs = len(durations)
    mean = sum(durations) / runs
    std = math.sqrt(sum((d - mean) ** 2 for d in durations) / max(1, runs - 1))
    return dict(runs=runs, mean=mean, std=std, err=std / math.sqrt(runs), best=float(min(durations)),
                worst=float(max(durations)))


def _check(data, out):
    """The package's check_implementation (same signature and tolerance as reference.py:275-283),
    given the expectation the literal port of the reference path computes on the GPUs over NCCL."""
    from gpu_mode_kernels_b200.all2all import check_implementation
    from oracle import a2a_oracle as O

    expected = O.port_ref_kernel(data, valid_rows_only=True)
    return check_implementation(data, out, expected)


def _run_case(rank, world, port, spec, mode, max_repeats, q):
    import torch.distributed as dist

    import gpu_mode_kernels_b200 as pkg
    from gpu_mode_kernels_b200.all2all import custom_kernel

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    result = None
    try:
        cfg, rd, _, _ = pkg.reference_task_input(spec, rank, world, device=f"cuda:{rank}")
        data = (cfg, rd, rank, world)
        torch.cuda.synchronize()
        dist.barrier()
        out = custom_kernel(data)
        torch.cuda.synchronize()
        good, message = _check(data, out)
        if mode == "test" or not good:
            result = (good, message)
        else:
            flush = torch.empty(256 << 20, dtype=torch.int8, device=f"cuda:{rank}")
            durations = []
            for i in range(max_repeats):
                flush.fill_(42)  # clear_l2_cache (utils.py:159-166)
                torch.cuda.synchronize()
                dist.barrier()
                t0 = time.perf_counter_ns()
                out = custom_kernel(data)
                torch.cuda.synchronize()
                dist.barrier()
                durations.append(time.perf_counter_ns() - t0)
                del out
            result = _stats(durations)
    except Exception as e:  # noqa: BLE001
        result = (False, repr(e))
    q.put((rank, result))
    if isinstance(result, tuple) and not result[0]:
        q.close()
        q.join_thread()
        os._exit(1)
    dist.destroy_process_group()  # releases this case's contexts (hook in all2all.py)


def run_case(world, port, spec, mode, max_repeats=50):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_run_case, args=(r, world, port, spec, mode, max_repeats, q), daemon=True)
             for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(30)
    return res


def main():
    import gpu_mode_kernels_b200 as pkg

    ap = argparse.ArgumentParser()
    ap.add_argument("action", choices=["test", "benchmark"])
    ap.add_argument("--world", type=int, default=min(8, torch.cuda.device_count()))
    ap.add_argument("--limit", type=int, default=None, help="only the first N cases")
    args = ap.parse_args()
    specs = pkg.REFERENCE_TESTS if args.action == "test" else pkg.REFERENCE_BENCHMARKS
    specs = [s for s in specs if s[0] % args.world == 0][: args.limit]
    print(f"{args.action}-count", len(specs))
    for idx, spec in enumerate(specs):
        res = run_case(args.world, 12356 + idx, spec, args.action)
        if args.action == "test":
            bad = [(r, v[1]) for r, v in sorted(res.items()) if not v[0]]
            print(f"test.{idx}.status", "fail" if bad else "pass")
            if bad:
                print(f"test.{idx}.error", "; ".join(f"rank {r} - {m}" for r, m in bad))
                break
        else:
            r0 = res[0]
            if isinstance(r0, dict):
                for k in ("runs", "mean", "std", "err", "best", "worst"):
                    print(f"benchmark.{idx}.{k}", r0[k])
            else:
                print(f"benchmark.{idx}.status", "fail")
                print(f"benchmark.{idx}.error", r0[1])


if __name__ == "__main__":
    main()
