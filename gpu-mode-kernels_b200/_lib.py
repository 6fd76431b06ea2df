"""ctypes binding of liba2a.so (the C ABI declared in include/a2a.h).

There is no fallback: if the library is missing or does not load, the first use
raises.  Build it with ``python gpu-mode-kernels_b200/build.py`` (or
``__graft_entry__.build()``).
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "liba2a.so")

A2A_OK, A2A_ERR_CONFIG, A2A_ERR_CAPACITY, A2A_ERR_TIMEOUT, A2A_ERR_STATE, A2A_ERR_ROUTING = range(6)
DTYPE_BF16, DTYPE_FP16 = 0, 1
PAYLOAD = {"direct": 0, "dedup": 1, "fp8": 2}
SCHEDULE = {"phased": 0, "pipelined": 1}
COMBINE = {"pull": 0, "push": 1}
MAX_WORLD, MAX_EXPERTS, MAX_TOPK = 8, 1024, 32


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "rank", "world_size", "device", "num_experts", "experts_per_token", "hidden_dim",
        "max_num_tokens", "dtype", "payload", "timeout_ms", "schedule", "combine", "chunks", "senders")]


class Status(C.Structure):
    _fields_ = [("code", C.c_int32), ("rank", C.c_int32), ("peer", C.c_int32), ("phase", C.c_int32),
                ("epoch", C.c_uint32), ("detail", C.c_int32)]


class A2AError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"a2a error {code}: {message}")
        self.code = code


# name -> (restype, argtypes); every symbol include/a2a.h declares
_VP, _I = C.c_void_p, C.c_int
SIGNATURES = {
    "a2a_strerror": (C.c_char_p, [_I]),
    "a2a_create": (_I, [C.POINTER(_VP), C.POINTER(Config)]),
    "a2a_destroy": (_I, [_VP]),
    "a2a_ipc_handle_bytes": (C.c_size_t, []),
    "a2a_export_handle": (_I, [_VP, _VP]),
    "a2a_open_peers": (_I, [_VP, _VP, C.c_size_t]),
    "a2a_last_error": (C.c_char_p, [_VP]),
    "a2a_fingerprint": (_I, [C.POINTER(Config), _VP]),
    "a2a_check_handles": (_I, [C.POINTER(Config), _VP, C.c_size_t, C.c_char_p, C.c_size_t]),
    "a2a_pipe_step": (_I, [_VP, _I, _VP, _VP, _VP, _VP, _I, _VP]),
    "a2a_attach_local_peers": (_I, [_VP, C.POINTER(_VP)]),
    "a2a_route": (_I, [_VP, _VP, _I, _VP]),
    "a2a_dispatch_send": (_I, [_VP, _VP, _VP]),
    "a2a_dispatch_recv": (_I, [_VP, _VP]),
    "a2a_expert_placeholder": (_I, [_VP, _VP]),
    "a2a_dispatch_recv_expert": (_I, [_VP, _VP]),
    "a2a_expert_done": (_I, [_VP, _VP]),
    "a2a_combine": (_I, [_VP, _VP, _VP, _VP]),
    "a2a_forward": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _VP]),
    "a2a_set_fused": (_I, [_VP, _I]),
    "a2a_forward_host": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _VP]),
    "a2a_barrier": (_I, [_VP, _VP]),
    "a2a_link_probe": (_I, [_VP, _I, C.c_size_t, _VP]),
    "a2a_export_dispatch": (_I, [_VP, _VP, _VP, _VP, _VP]),
    "a2a_expert_buffers": (_I, [_VP, C.POINTER(_VP), C.POINTER(_VP)]),
    "a2a_route_buffers": (_I, [_VP, C.POINTER(_VP), C.POINTER(_VP)]),
    "a2a_copy_route": (_I, [_VP, _VP, _VP, _VP]),
    "a2a_route_noalloc": (_I, [_VP, _I, _I, _I, _VP, _VP, _VP]),
    "a2a_histogram256": (_I, [_VP, C.c_size_t, _VP, _VP]),
    "a2a_status": (_I, [_VP, C.POINTER(Status)]),
    "a2a_status_clear": (_I, [_VP]),
    "a2a_status_peek": (_I, [_VP]),
    "a2a_trace_enable": (_I, [_VP, _I]),
    "a2a_trace_read": (_I, [_VP, _VP, _I, C.POINTER(_I), C.POINTER(_I)]),
    "a2a_launch_count": (C.c_int64, [_VP]),
    "a2a_symmetric_bytes": (C.c_size_t, [_VP]),
}

_lib = None


def load() -> C.CDLL:
    """Load liba2a.so once and type its entry points; raise if it is not there."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(run `python gpu-mode-kernels_b200/build.py`); there is no CPU fallback")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def strerror(code: int) -> str:
    return load().a2a_strerror(code).decode()


def check(code: int) -> None:
    if code != 0:
        raise A2AError(code, strerror(code))
