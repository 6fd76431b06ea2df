"""CPU-only checks of bench.py's reference arm (the port of the reference path under gloo)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _last_json(out: str):
    lines = [l for l in out.splitlines() if l.startswith("{")]
    assert lines, out
    return json.loads(lines[-1])


def test_reference_arm_prints_the_contract_line_single_rank():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    d = _last_json(res.stdout)
    assert d["impl"] == "reference" and d["unit"] == "us" and d["higher_is_better"] is False
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"].startswith("c1:")


def test_reference_arm_under_torchrun_two_ranks_rank0_only_prints():
    """Launched like the driver launches N > 1: rank 0 runs the CPU ranks itself (private rendezvous,
    the launcher's TORCHELASTIC_* variables must not leak into it), the other rank exits quietly."""
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29577", os.path.join(ROOT, "bench.py"),
                          "--impl", "reference", "--gpus", "2", "--workload", "c1", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["n_gpus"] == 2 and d["config"]["world_size"] == 2 and "2 gloo process" in d["cpu_baseline"]["sample"]


def test_reference_arm_of_the_histogram_workload():
    """`--workload histogram --impl reference`: the reference's own operator call timed on the host cores."""
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload",
                          "histogram", "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    d = _last_json(res.stdout)
    assert d["impl"] == "reference" and d["metric"] == "histogram us" and d["dtype"] == "u8" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "reference" and "bincount" in d["cpu_baseline"]["sample"]
