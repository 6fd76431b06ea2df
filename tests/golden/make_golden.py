"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself.

Run where the reference checkout is available, pointing ``A2A_REFERENCE_DIR`` at it:

    A2A_REFERENCE_DIR=/path/to/gpu-mode-kernels python tests/golden/make_golden.py

For every case below it starts ``world_size`` CPU processes on the gloo
backend, imports the unmodified ``reference.py`` of
``amd-distributed/all2all`` and records, per rank, the inputs and what
``PyTorchAllToAll.dispatch`` and ``ref_kernel`` returned (the valid prefix of
every expert only: the reference leaves the padding uninitialised).  16-bit
floats are stored as their raw bit patterns (uint16).  The inputs come from this
repository's CPU generator, because the reference's own ``generate_input`` needs
a CUDA device.
"""
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if "A2A_REFERENCE_DIR" not in os.environ:
    sys.exit("set A2A_REFERENCE_DIR to the checkout of gau-nernst/gpu-mode-kernels")
REF_DIR = os.path.join(os.environ["A2A_REFERENCE_DIR"], "amd-distributed", "all2all")

# name -> (world_size, generate_input kwargs)
CASES = {
    # the CPU-runnable configuration the metric's config list starts with
    "c1_ws2_bf16": (2, dict(num_experts=8, experts_per_token=2, hidden_dim=2048, max_num_tokens=16, seed=0)),
    "ws1_bf16": (1, dict(num_experts=8, experts_per_token=3, hidden_dim=64, max_num_tokens=5, seed=11)),
    "ws4_bf16_ragged": (4, dict(num_experts=16, experts_per_token=4, hidden_dim=256, max_num_tokens=8, seed=7,
                                ragged=True)),
    "ws8_bf16_zipf": (8, dict(num_experts=64, experts_per_token=6, hidden_dim=128, max_num_tokens=8, seed=2,
                              routing="zipf")),
    # the reference task's own style: fp16, uniform weights, random token count, H=2880
    "ws2_fp16_task": (2, dict(num_experts=8, experts_per_token=2, hidden_dim=2880, max_num_tokens=6, seed=347,
                              dtype="float16", weights="rand", ragged=True)),
    "ws8_fp16_task": (8, dict(num_experts=128, experts_per_token=8, hidden_dim=64, max_num_tokens=16, seed=175,
                              dtype="float16", weights="rand", ragged=True)),
}


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _worker(rank: int, ws: int, kwargs: dict, port: int, outdir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    sys.path.insert(0, REF_DIR)
    sys.path.insert(0, ROOT)
    import reference as R  # the unmodified reference (imports its own task.py)
    import gpu_mode_kernels_b200 as pkg

    kw = dict(kwargs)
    dtype = getattr(torch, kw.pop("dtype", "bfloat16"))
    cfg, rd, _, _ = pkg.generate_input(rank=rank, world_size=ws, dtype=dtype, **kw)
    rcfg = R.MoEConfig(num_experts=cfg.num_experts, experts_per_token=cfg.experts_per_token,
                       hidden_dim=cfg.hidden_dim, max_num_tokens=cfg.max_num_tokens,
                       in_dtype=dtype, out_dtype=dtype)
    ata = R.PyTorchAllToAll(rcfg, rank, ws)
    n, ex, em = ata.dispatch(rd.x, rd.indices)
    y = R.ref_kernel((rcfg, rd, rank, ws))
    rows = torch.cat([ex[e, : int(n[e])] for e in range(n.numel())], 0)
    meta = torch.cat([em[e, : int(n[e])] for e in range(n.numel())], 0)
    np.savez(os.path.join(outdir, f"r{rank}.npz"),
             indices=rd.indices.numpy(), weights=rd.weights.numpy(), x=_bits(rd.x),
             num_tokens=np.int64(rd.num_tokens),
             expert_num_tokens=n.numpy(), rows=_bits(rows), meta=meta.numpy(), y=_bits(y))
    dist.barrier()
    dist.destroy_process_group()


def main():
    port = 29640
    for name, (ws, kwargs) in CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            mp.spawn(_worker, args=(ws, kwargs, port, tmp), nprocs=ws, join=True)
            port += 1
            out = {"world_size": np.int64(ws)}
            for key, val in kwargs.items():
                out[f"cfg_{key}"] = np.array(val)
            for r in range(ws):
                with np.load(os.path.join(tmp, f"r{r}.npz")) as z:
                    for key in z.files:
                        out[f"r{r}_{key}"] = z[key]
            path = os.path.join(HERE, f"{name}.npz")
            np.savez_compressed(path, **out)
            print(f"{name}: ws={ws} -> {path} ({os.path.getsize(path)} bytes)")


if __name__ == "__main__":
    main()
