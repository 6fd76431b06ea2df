"""CPU-side checks of the C-ABI boundary: the library loads, exports every declared symbol,
and rejects bad configurations before touching a device."""
import ctypes as C
import os
import re

import pytest

import gpu_mode_kernels_b200 as pkg
from gpu_mode_kernels_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "a2a.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(a2a_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/a2a.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_strerror_and_handle_size():
    lib = _lib.load()
    assert lib.a2a_ipc_handle_bytes() == 128  # 64-byte CUDA IPC handle + configuration fingerprint
    assert _lib.strerror(0) == "ok"
    for code in range(1, 6):
        assert _lib.strerror(code) not in ("ok", "unknown status")


@pytest.mark.parametrize("kw", [
    dict(world_size=0), dict(world_size=9), dict(rank=2), dict(num_experts=7), dict(num_experts=2048),
    dict(experts_per_token=0), dict(experts_per_token=33), dict(hidden_dim=100), dict(hidden_dim=0),
    dict(max_num_tokens=0), dict(dtype=5), dict(payload=7), dict(device=-1),
    dict(schedule=2), dict(combine=3), dict(chunks=9), dict(senders=-1),
    dict(schedule=1, payload=0),            # the pipelined schedule moves (token, rank) wire rows: needs DEDUP
    dict(schedule=0, payload=1, combine=1),  # expert-side reduction exists in the pipelined schedule only
    dict(schedule=1, payload=1, chunks=2),
    dict(schedule=1, payload=1, senders=1),  # two sender blocks carry the watchers
])
def test_bad_config_is_rejected_without_a_device(kw):
    lib = _lib.load()
    base = dict(rank=0, world_size=2, device=0, num_experts=8, experts_per_token=2, hidden_dim=64,
                max_num_tokens=4, dtype=0, payload=0, timeout_ms=100)
    base.update(kw)
    cfg = _lib.Config(**base)
    h = C.c_void_p()
    assert lib.a2a_create(C.byref(h), C.byref(cfg)) == _lib.A2A_ERR_CONFIG
    assert not h.value


def test_null_arguments():
    lib = _lib.load()
    assert lib.a2a_create(None, None) == _lib.A2A_ERR_CONFIG
    assert lib.a2a_destroy(None) == 0
    assert lib.a2a_route(None, None, 0, None) == _lib.A2A_ERR_CONFIG
    assert lib.a2a_launch_count(None) == 0
