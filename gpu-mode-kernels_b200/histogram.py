"""Host side of the byte histogram: the plugin entry of the reference's second task.

``custom_kernel((data, output))`` has the signature the task defines
(pmpp_v2/histogram_py/task.py:4-5; submission entry pmpp_v2/histogram_py/submission_v1.py:110-113):
``data`` uint8 ``[size]`` on the GPU, ``output`` int64 ``[256]`` preallocated by the caller; the counts
are written into ``output`` and it is returned.  All work is in liba2a.so (``a2a_histogram256``);
there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch

from . import _lib

NUM_BINS = 256


def histogram256(data: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
    """Counts of the byte values of ``data`` into ``output`` on the current stream; returns ``output``."""
    if data.dtype != torch.uint8 or not data.is_cuda or not data.is_contiguous() or data.dim() != 1:
        raise _lib.A2AError(_lib.A2A_ERR_CONFIG, f"data must be a contiguous 1-D uint8 CUDA tensor, got {data.dtype} {tuple(data.shape)} on {data.device}")
    if (output.dtype != torch.int64 or output.numel() != NUM_BINS or not output.is_contiguous()
            or output.device != data.device):
        raise _lib.A2AError(_lib.A2A_ERR_CONFIG, f"output must be a contiguous int64 [{NUM_BINS}] tensor on {data.device}")
    lib = _lib.load()
    with torch.cuda.device(data.device):
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(lib.a2a_histogram256(C.c_void_p(data.data_ptr()), data.numel(), C.c_void_p(output.data_ptr()), stream))
    return output


def custom_kernel(data: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    values, output = data
    return histogram256(values, output)
