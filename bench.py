#!/usr/bin/env python
"""Benchmark of the MoE all-to-all path: dispatch + expert placeholder + combine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4]

One process per GPU (N > 1: launched by ``python -m torch.distributed.run``; rank,
world size and rendezvous come from the environment).  A step is one
``custom_kernel`` forward of every rank on the 256-expert / top-8 / hidden 7168 /
256 tokens-per-rank bf16 workload with the experts split evenly over the N ranks.
Rank 0 prints ONE JSON line.

Timed region (``value``): inputs resident in HBM; per step an untimed L2 flush
(256 MiB write) and, for N > 1, a device-side rendezvous of all ranks, then CUDA
events on the launching stream around the forward; a step costs the maximum over
ranks; the K steps are enqueued back to back with a synchronise and barrier on
both sides of the loop.  ``e2e`` times the same step through the host-buffer entry
point (pinned host tensors in, pinned host tensor out, copies inside the events).
``--impl reference`` times the CPU restatement of the reference's Python path
(oracle/, gloo, one process per rank on the host cores).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "dispatch+combine us (max over ranks)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4")
    ap.add_argument("--payload", default=None, help="direct | dedup | fp8 (default: the workload's own)")
    ap.add_argument("--schedule", default=None, help="pipelined | phased (default: pipelined where the payload allows)")
    ap.add_argument("--combine", default=None, help="push | pull (default: push with the pipelined schedule)")
    ap.add_argument("--senders", type=int, default=0, help="sender blocks of the pipelined kernel (0: library default)")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true",
                    help="skip the check of one forward of every rank (dispatch digests and outputs) against the CPU checker")
    ap.add_argument("--skip-link-probe", action="store_true")
    ap.add_argument("--no-l2-flush", action="store_true",
                    help="diagnostic only: leave the L2 warm between steps (such a number breaks the timing rules and "
                         "is labelled so in config.l2)")
    ap.add_argument("--trace", default=None, help="write the merged in-kernel trace of one forward (chrome JSON) here")
    ap.add_argument("--per-phase-launches", action="store_true",
                    help="phased schedule: run the forward as one kernel per phase instead of one cooperative launch")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed loop runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self.nv = None

    def _names(self, mask: int):
        nv = self.nv
        table = {
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        return [n for n, bit in table.items() if mask & bit]

    def _run(self):
        nv = self.nv
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                if get_reasons is not None:
                    self.reasons.update(self._names(int(get_reasons(self.h))))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(1.0)

    def summary(self):
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:  # noqa: BLE001
            return local_index
    return local_index


# ---------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's Python path, under gloo
# ---------------------------------------------------------------------------
def _ref_rank(rank, ws, port, workload, steps, warmup, threads, q):
    import torch.distributed as dist

    import gpu_mode_kernels_b200 as pkg
    from oracle import a2a_oracle as O

    # a private TCP rendezvous: under torchrun the inherited TORCHELASTIC_* variables would make an
    # env:// rendezvous look for the launcher's store instead of starting ours
    for k in [k for k in os.environ if k.startswith("TORCHELASTIC_")]:
        os.environ.pop(k)
    torch.set_num_threads(threads)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=ws)
    cfg, rd, _, _ = pkg.workload_input(workload, rank, ws)
    ata = O.PortAllToAll(cfg, rank, ws)
    full_tokens = rd.num_tokens
    budget_s = float(os.environ.get("A2A_REFERENCE_BUDGET_S", "150"))

    def one_step(n_tok):
        x, idx, w = rd.x[:n_tok], rd.indices[:n_tok], rd.weights[:n_tok]
        dist.barrier()
        t0 = time.perf_counter()
        n, ex, em = ata.dispatch(x, idx)
        t1 = time.perf_counter()
        ey = O.port_expert_op(ex, cfg.out_dtype, rank, n)  # valid rows only; not part of the metric
        t2 = time.perf_counter()
        y = torch.zeros(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype)
        ata.combine(y, w, em, ey, n)
        t3 = time.perf_counter()
        t = torch.tensor([(t1 - t0) + (t3 - t2), t2 - t1], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1])

    # One full-size probe step decides whether the steps can be full size within the
    # time budget; if not, every step runs on the first n_tok tokens of each rank and
    # its time is scaled by full_tokens / n_tok (the Python loops are linear in tokens).
    probe, _ = one_step(full_tokens)
    n_tok = full_tokens
    if probe * (steps + warmup) > budget_s:
        n_tok = max(8, int(full_tokens * budget_s / (probe * (steps + warmup))))
    scale = full_tokens / n_tok
    times, expert_s = [], []
    for it in range(warmup + steps):
        a, b = one_step(n_tok)
        if it >= warmup:
            times.append(a * scale)
            expert_s.append(b * scale)
    if rank == 0:
        q.put((times, expert_s, n_tok, full_tokens))
    dist.barrier()
    dist.destroy_process_group()


def run_reference_cpu(ws: int, workload: str, steps: int, warmup: int):
    """dispatch+combine seconds per step (max over CPU ranks) of the port; all host threads."""
    import torch.multiprocessing as mp

    cores = os.cpu_count() or 1
    threads = max(1, cores // ws)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 50)
    procs = [ctx.Process(target=_ref_rank, args=(r, ws, port, workload, steps, warmup, threads, q)) for r in range(ws)]
    for p in procs:
        p.start()
    times, expert_s, n_tok, full_tokens = q.get(timeout=3600)
    for p in procs:
        p.join(120)
    return times, expert_s, cores, threads, (n_tok, full_tokens)


def reference_main(args, rank: int, ws: int):
    if rank != 0:
        return
    times, expert_s, cores, threads, (n_tok, full_tokens) = run_reference_cpu(ws, args.workload, args.steps, args.warmup)
    us = 1e6 * sum(times) / len(times)
    what = "full" if n_tok == full_tokens else f"first {n_tok} of {full_tokens} tokens per rank (time scaled by {full_tokens / n_tok:.2f}) of the"
    sample = (f"{what} {args.workload} workload at world size {ws}, {ws} gloo process(es) x {threads} torch thread(s); "
              f"dispatch+combine wall clock between barriers, max over ranks; the expert placeholder "
              f"(valid rows only, {1e3 * sum(expert_s) / len(expert_s):.1f} ms) is not counted")
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us", "n_gpus": ws, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, ws, "n/a (CPU)", "n/a (CPU)"),
        "cpu_baseline": {"value": us, "unit": "us", "cores": min(cores, ws * threads), "kind": "port", "sample": sample},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name: str, ws: int, payload: str, launches: str = "one cooperative launch per forward"):
    import gpu_mode_kernels_b200 as pkg

    w = pkg.WORKLOADS[name]
    return {
        "workload": f"{name}: {w['num_experts']} experts ({w['num_experts'] // ws} per rank), top-{w['experts_per_token']}, "
                    f"hidden {w['hidden_dim']}, {w['max_num_tokens']} tokens/rank, bf16, "
                    f"{w.get('routing', 'uniform')} routing, softmax weights, seed {w['seed']}",
        "world_size": ws, "payload": payload, "launches": launches,
        "global_tokens": w["max_num_tokens"] * ws,
        "l2": "flushed between timed steps (256 MiB write, untimed)",
    }


def percentile(values, q):
    v = sorted(values)
    return v[min(len(v) - 1, int(round(q * (len(v) - 1))))]


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def main():
    args = parse_args()
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if ws == 1 and args.gpus > 1:
        sys.exit("bench.py --gpus N>1 must be launched with python -m torch.distributed.run --nproc-per-node N")
    if args.workload == "histogram":
        histogram_main(args, rank, ws)
        return
    if args.impl == "reference":
        reference_main(args, rank, ws)
        return

    import torch.distributed as dist

    import gpu_mode_kernels_b200 as pkg
    from gpu_mode_kernels_b200 import traffic, verify
    from gpu_mode_kernels_b200.all2all import A2AContext

    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if ws > 1:
        # keep stdout to the one JSON line: NCCL's version banner (NCCL_DEBUG=VERSION) goes there too
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=dev)

    wl = pkg.WORKLOADS[args.workload]
    payload = args.payload or wl.get("payload", "dedup")
    schedule = args.schedule or ("pipelined" if payload in ("dedup", "fp8") else "phased")
    combine = args.combine or ("push" if schedule == "pipelined" else "pull")
    cfg, rd_cpu, _, _ = pkg.workload_input(args.workload, rank, ws)
    rd = rd_cpu.to(dev)
    T, K, H = rd.num_tokens, cfg.experts_per_token, cfg.hidden_dim
    ctx = A2AContext(cfg, rank, ws, device=local_rank, payload=payload, schedule=schedule, combine=combine,
                     senders=args.senders)
    pipelined = schedule == "pipelined"
    if args.per_phase_launches and not pipelined:
        ctx.set_fused(False)
    fused = pipelined or not args.per_phase_launches
    y = torch.empty(T, H, dtype=cfg.out_dtype, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.int8, device=dev)
    stream = torch.cuda.current_stream()

    def sync_all():
        torch.cuda.synchronize()
        if ws > 1:
            dist.barrier()

    def max_over_ranks(ms_list):
        t = torch.tensor(ms_list, dtype=torch.float64, device=dev)
        if ws > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.cpu().tolist()

    def timed_loop(step_fn, steps, warmup):
        for i in range(warmup):
            if not args.no_l2_flush:
                flush.fill_(i & 1)
            if ws > 1:
                ctx.barrier()
            step_fn()
        sync_all()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        l0 = ctx.launches
        for i in range(steps):
            if not args.no_l2_flush:
                flush.fill_(i & 1)
            if ws > 1:
                ctx.barrier()
            ev[i][0].record(stream)
            step_fn()
            ev[i][1].record(stream)
        sync_all()
        launches = ctx.launches - l0
        return max_over_ranks([a.elapsed_time(b) for a, b in ev]), launches

    # ---- headline: device-resident inputs --------------------------------
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        per_step_ms, launches = timed_loop(lambda: ctx.forward(rd.x, rd.indices, rd.weights, y), args.steps, args.warmup)
    ctx.check()
    ms = sum(per_step_ms) / len(per_step_ms)
    if ws > 1:
        launches -= args.steps  # the device-side rendezvous before every step is not part of the path

    # ---- end to end: host buffers through the plugin-facing entry --------
    hx, hi, hw = rd_cpu.x.pin_memory(), rd_cpu.indices.pin_memory(), rd_cpu.weights.pin_memory()
    hy = torch.empty(T, H, dtype=cfg.out_dtype, pin_memory=True)
    e2e_steps = min(args.steps, 200)
    e2e_ms_list, _ = timed_loop(lambda: ctx.forward_host(hx, hi, hw, hy), e2e_steps, min(args.warmup, 10))
    ctx.check()
    e2e_ms = sum(e2e_ms_list) / len(e2e_ms_list)
    h2d = hx.numel() * hx.element_size() + hi.numel() * 4 + hw.numel() * 4
    d2h = hy.numel() * hy.element_size()

    # ---- per-kernel pass: events between the separate launches of the same device code ----
    ph_steps = min(args.steps, 200)
    if pipelined:
        names = ["send_route", "expert", "combine"]
        calls = [lambda: ctx.pipe_step(0, rd.x, rd.indices, rd.weights, y), lambda: ctx.pipe_step(1),
                 lambda: ctx.pipe_step(2)]
    else:
        names = ["route", "dispatch_send", "recv_expert", "combine"]
        calls = [lambda: ctx.route(rd.indices), lambda: ctx.dispatch_send(rd.x), ctx.dispatch_recv_expert,
                 lambda: ctx.combine(rd.weights, y)]
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(ph_steps)]
    for i in range(ph_steps + 5):
        flush.fill_(i & 1)
        if ws > 1:
            ctx.barrier()
        e = evs[i - 5] if i >= 5 else None
        for j, fn in enumerate(calls):
            if e: e[j].record(stream)
            fn()
        if e: e[len(calls)].record(stream)
    sync_all()
    ctx.check()
    phase_us = {}
    for j, n in enumerate(names):
        per = max_over_ranks([e[j].elapsed_time(e[j + 1]) for e in evs])
        phase_us[n] = 1e3 * sum(per) / len(per)

    # ---- measured peer-copy bandwidth of this box (every rank copies to its neighbour at once) ----
    link = None
    if ws > 1 and not args.skip_link_probe:
        nbytes = min(256 << 20, T * ws * (cfg.num_experts // ws) * H * 2)
        reps = 10
        for _ in range(2):
            ctx.link_probe((rank + 1) % ws, nbytes)
        sync_all()
        ctx.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            ctx.link_probe((rank + 1) % ws, nbytes)
        b.record(stream)
        sync_all()
        t_ms = max_over_ranks([a.elapsed_time(b)])[0]
        link = {"peer_copy_gbs": nbytes * reps / (t_ms * 1e-3) / 1e9, "bytes": nbytes, "copies": reps,
                "how": "cudaMemcpyAsync device-to-device into the next rank's region, all ranks at once, CUDA events, "
                       "max over ranks"}

    # ---- traffic and roofline --------------------------------------------
    hbm_peak, peak_kind = measured_peaks()
    all_idx = [pkg.workload_input(args.workload, r, ws)[1].indices for r in range(ws)] if ws > 1 else [rd_cpu.indices]
    tr = traffic.summarize(all_idx, cfg.num_experts, ws, H, payload, combine)
    if ws == 1:
        alg = (3 * T * K + T) * 2 * H  # rows written and read in dispatch, read in combine, y written
        achieved = alg / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "one-launch forward (route + send + expert + combine)",
                    "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                    "traffic": SINGLE_GPU_TRAFFIC.get((args.workload, schedule, combine)),
                    "peak_kind": f"of {peak_kind}", "algorithmic_bytes": alg, "kernel_us": ms * 1e3,
                    "traffic_note": "bytes per launch from one ncu capture of this kernel on this workload "
                                    "(dram__bytes_read.sum + dram__bytes_write.sum; L2 traffic beside it): the working set "
                                    "fits the 126 MB L2, so DRAM sees far less than the algorithmic bytes"}
        nvlink = None
    else:
        achieved = tr["algorithmic_bytes"] / (ms * 1e-3) / 1e9
        roofline = {"bound": "nvlink", "kernel": "one-launch forward (dispatch + combine transfers)", "achieved": achieved,
                    "peak": traffic.NVLINK_NOMINAL_GBS, "unit": "GB/s", "frac": achieved / traffic.NVLINK_NOMINAL_GBS,
                    "traffic": None, "peak_kind": "of nominal NVLink 5 per direction (900 GB/s)",
                    "algorithmic_bytes": tr["algorithmic_bytes"], "wire_bytes": tr["wire_bytes"],
                    "wire_gbs": tr["wire_bytes"] / (ms * 1e-3) / 1e9,
                    "wire_frac": tr["wire_bytes"] / (ms * 1e-3) / 1e9 / traffic.NVLINK_NOMINAL_GBS}
        nvlink = {"algorithmic_gbs": achieved, "frac_of_900": achieved / traffic.NVLINK_NOMINAL_GBS,
                  "wire_gbs": roofline["wire_gbs"], "busiest_rows": tr["busiest_rows"],
                  "busiest_rows_dedup": tr["busiest_rows_dedup"], "t_roof_us_900": tr["t_roof_us_nominal"],
                  "t_wire_us_900": tr["t_wire_us_nominal"], "measured_link": link}

    # ---- CPU baseline (rank 0, N=1 only): the port of the reference path --
    cpu_baseline = None
    if ws == 1 and not args.skip_cpu_baseline:
        times, expert_s, cores, threads, _ = run_reference_cpu(1, args.workload, 3, 1)
        cpu_baseline = {"value": 1e6 * min(times), "unit": "us", "cores": threads, "kind": "port",
                        "sample": f"full {args.workload} workload at world size 1, one gloo process with {threads} torch "
                                  f"threads; dispatch+combine of the reference's Python path, best of 3; expert "
                                  f"placeholder on valid rows ({1e3 * min(expert_s):.1f} ms) not counted"}

    # ---- parity of the path that was just timed: one more forward of every rank, checked on rank 0 ----
    verified = None
    if not args.no_verify:
        yv = ctx.forward(rd.x, rd.indices, rd.weights)
        sync_all()
        ctx.check()
        counts, rows, meta = ctx.export_dispatch()
        torch.cuda.synchronize()
        crows, cmeta = verify.compact_dispatch(counts.cpu(), rows, meta)
        digest = torch.tensor(verify.dispatch_digest(counts.cpu(), crows, cmeta), dtype=torch.int64, device=dev)
        del rows, meta, crows, cmeta
        gathered = [torch.empty_like(yv) for _ in range(ws)] if rank == 0 else None
        digests = [torch.empty_like(digest) for _ in range(ws)] if rank == 0 else None
        if ws > 1:
            dist.gather(yv, gathered, dst=0)
            dist.gather(digest, digests, dst=0)
        else:
            gathered, digests = [yv], [digest]
        if rank == 0:
            from oracle import a2a_oracle as O

            rds = [pkg.workload_input(args.workload, r, ws)[1] for r in range(ws)]
            disp, ys = O.simulate(cfg, ws, rds)
            tol = 6e-2 if payload == "fp8" else 2e-2
            worst, outliers, dispatch_ok = 0.0, 0, True
            for r in range(ws):
                d = (gathered[r].cpu().float() - ys[r].float()).abs() / (tol + tol * ys[r].float().abs())
                worst = max(worst, float(d.max()))
                outliers += int((d > 1).sum())
                # the one-launch kernels leave the expert OUTPUT of every dispatched row in the slabs:
                # dtype(float(row) * (1 + rank)), one rounding (FP8: of the dequantised row)
                erows = disp[r].rows
                if payload == "fp8" and erows.numel():
                    q, sc = O.fp8_quantise(erows)
                    erows = O.fp8_dequantise(q, sc, cfg.in_dtype)
                erows = (erows.float() * float(1 + r)).to(cfg.in_dtype)
                want = verify.dispatch_digest(disp[r].expert_num_tokens, erows, disp[r].meta)
                dispatch_ok = dispatch_ok and tuple(int(v) for v in digests[r].cpu().tolist()) == want
            verified = {"ok": bool(dispatch_ok and worst <= (1.25 if payload == "fp8" else 1.0)),
                        "dispatch_bit_exact": bool(dispatch_ok), "rtol_atol": tol, "worst_diff_over_tol": worst,
                        "elements_outside": outliers,
                        "how": "one forward of every rank after the timed loops: digests of counts / rows / "
                               "(expert, source, token, k) records of every rank's slabs against the CPU checker's "
                               "dispatch, outputs against its combine"}
        sync_all()

    # ---- in-kernel trace of one forward, merged over the ranks -----------
    if args.trace:
        from gpu_mode_kernels_b200 import trace as tracing

        ctx.trace_enable(True)
        sync_all()
        # Two L2 flushes (~70 us each) keep the GPU busy while the host queues the rendezvous and the forward
        # behind them: when the rendezvous lets go, every rank's forward is already waiting in its stream, so
        # the ranks start within a microsecond or two of each other -- as they do in the timed loop.
        flush.fill_(0)
        flush.fill_(1)
        if ws > 1:
            ctx.barrier()
        ctx.forward(rd.x, rd.indices, rd.weights, y)
        stamps = ctx.trace_read()
        ctx.trace_enable(False)
        mine = tracing.rank_events(stamps, rank, sm_mhz=clocks.summary()["sm_mhz"] or 1965.0, world_size=ws,
                                   pipelined=pipelined)
        everyone = [None] * ws
        if ws > 1:
            dist.gather_object(mine, everyone if rank == 0 else None, dst=0)
        else:
            everyone = [mine]
        if rank == 0:
            tracing.write_chrome_trace(args.trace, everyone)
            with open(os.path.splitext(args.trace)[0] + "_summary.txt", "w") as f:
                f.write(tracing.summarize(everyone))
        sync_all()

    if rank == 0:
        line = {
            "metric": METRIC, "value": ms * 1e3, "unit": "us", "n_gpus": ws, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(args.workload, ws, payload,
                                      "one cooperative launch per forward" if fused else "one kernel per phase"),
            "roofline": roofline, "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "clocks": clocks.summary(),
            "kernels_us": phase_us, "tokens_per_s": T * ws / (ms * 1e-3),
            "p50_us": 1e3 * statistics.median(per_step_ms), "p95_us": 1e3 * percentile(per_step_ms, 0.95),
            "max_us": 1e3 * max(per_step_ms),
        }
        line["config"]["schedule"] = schedule
        line["config"]["combine"] = combine
        if args.no_l2_flush:
            line["config"]["l2"] = "NOT flushed between steps (diagnostic run; not a contract number)"
        if nvlink is not None:
            line["nvlink"] = nvlink
        if verified is not None:
            line["verified"] = verified
        print(json.dumps(line), flush=True)

    sync_all()
    ctx.close()
    if ws > 1:
        dist.destroy_process_group()
    if verified is not None and rank == 0 and not verified["ok"]:
        sys.exit(3)


def histogram_main(args, rank: int, ws: int):
    """`--workload histogram`: the reference repository's second task (pmpp_v2/histogram_py) on its
    largest benchmark case, 10 485 760 bytes at 10 % contention (task.yml:39).  Does not shard: with
    N > 1 every rank runs its own replica ("replicas only"); rank 0 reports one replica's time."""
    if rank != 0:
        return
    from oracle import histogram_oracle as HO

    size, seed, contention = HO.REFERENCE_BENCHMARKS[-1]
    data_cpu, _ = HO.generate_input(size, contention, seed)
    if args.impl == "reference":
        torch.set_num_threads(os.cpu_count() or 1)
        times = []
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            torch.bincount(data_cpu, minlength=256)  # the reference's own call (reference.py:17), on the host cores
            if i >= args.warmup:
                times.append(time.perf_counter() - t0)
        us = 1e6 * sum(times) / len(times)
        print(json.dumps({"impl": "reference", "metric": "histogram us", "value": us, "unit": "us", "n_gpus": ws,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
                          "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                          "config": {"workload": f"histogram: {size} bytes, contention {contention} %, seed {seed}"},
                          "cpu_baseline": {"value": us, "unit": "us", "cores": torch.get_num_threads(), "kind": "reference",
                                           "sample": "torch.bincount(data, minlength=256) on the full input"},
                          "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0}), flush=True)
        return
    from gpu_mode_kernels_b200.histogram import histogram256

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    data = data_cpu.to(dev)
    out = torch.empty(256, dtype=torch.int64, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.int8, device=dev)
    stream = torch.cuda.current_stream()

    def loop(fn, steps, warmup):
        for i in range(warmup):
            flush.fill_(i & 1)
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for i in range(steps):
            flush.fill_(i & 1)
            ev[i][0].record(stream)
            fn()
            ev[i][1].record(stream)
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in ev]

    with ClockSampler(physical_gpu_index(0)) as clocks:
        ms_list = loop(lambda: histogram256(data, out), args.steps, args.warmup)
    ok = bool(torch.equal(out.cpu(), HO.ref_histogram(data_cpu)))
    ms = sum(ms_list) / len(ms_list)
    host = data_cpu.pin_memory()
    host_out = torch.empty(256, dtype=torch.int64, pin_memory=True)

    def e2e():
        data.copy_(host, non_blocking=True)
        histogram256(data, out)
        host_out.copy_(out, non_blocking=True)

    e2e_ms = loop(e2e, min(args.steps, 100), 5)
    hbm_peak, peak_kind = measured_peaks()
    alg = size + 256 * 8
    t0 = time.perf_counter()
    for _ in range(5):
        torch.bincount(data_cpu, minlength=256)
    cpu_us = 1e6 * (time.perf_counter() - t0) / 5
    print(json.dumps({
        "metric": "histogram us", "value": ms * 1e3, "unit": "us", "n_gpus": ws, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": f"histogram: {size} bytes, contention {contention} %, seed {seed}; replicas only",
                   "l2": "flushed between timed steps (256 MiB write, untimed)"},
        "roofline": {"bound": "hbm", "kernel": "histogram256_kernel (+ 2 KB memset)", "achieved": alg / (ms * 1e-3) / 1e9,
                     "peak": hbm_peak, "unit": "GB/s", "frac": alg / (ms * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                     "peak_kind": f"of {peak_kind}", "algorithmic_bytes": alg},
        "cpu_baseline": {"value": cpu_us, "unit": "us", "cores": torch.get_num_threads(), "kind": "reference",
                         "sample": "torch.bincount(data, minlength=256) on the full input, mean of 5"},
        "e2e": {"value": 1e3 * sum(e2e_ms) / len(e2e_ms), "unit": "us", "h2d_bytes_per_step": size, "d2h_bytes_per_step": 2048},
        "gpu_launches": args.steps, "clocks": clocks.summary(), "verified": {"ok": ok, "how": "counts equal torch.bincount on the CPU"},
        "p50_us": 1e3 * statistics.median(ms_list), "p95_us": 1e3 * percentile(ms_list, 0.95),
    }), flush=True)
    if not ok:
        sys.exit(3)


# DRAM and L2 bytes per launch of the one-launch kernel at world size 1, from ncu captures of this
# kernel on this workload (a profiler cannot run inside the timed loop, so the figures are constants
# of the kernel + workload, re-measured whenever the kernel changes).
SINGLE_GPU_TRAFFIC = {
    ("c4", "pipelined", "push"): {"dram_bytes": 5.26e6, "l2_bytes": 37.0e6,
                                  "source": "ncu --set full, pipe_forward_kernel, c4 at world size 1: dram__bytes_read.sum 3.79 MB + "
                                            "dram__bytes_write.sum 1.46 MB; L2 sectors from the SMs 3.93 MB read + 33.1 MB written"},
    ("c4", "phased", "pull"): {"dram_bytes": 7.76e6, "l2_bytes": 100.2e6,
                               "source": "ncu --set full, forward_kernel (phased schedule), c4 at world size 1: dram__bytes_read.sum "
                                         "4.16 MB + dram__bytes_write.sum 3.60 MB; L2 sectors from the SMs 63.4 MB read + 36.8 MB written"},
}


if __name__ == "__main__":
    main()
