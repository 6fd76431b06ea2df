"""Host side of the path: per-group context and the ``custom_kernel`` plugin entry.

``A2AContext`` plays the role of ``P2PState`` in the reference's final submission
(amd-distributed/all2all/submission_v9.py:880-947): it owns this rank's symmetric
receive region, exchanges one handle blob per rank with a single ``all_gather``
(NCCL or gloo -- the only collective this package ever issues) and maps the
peers.  ``custom_kernel(data)`` has the signature the task defines
(task.py:8-9, submission_v9.py:976-982): ``data = (cfg, rank_data, rank,
world_size)`` in, ``[num_tokens, hidden_dim]`` tensor of ``cfg.out_dtype`` out.
All compute is in liba2a.so; nothing here has a CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib
from ._lib import A2AError, Config, Status  # noqa: F401
from .task import MoEConfig, input_t, output_t

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


class A2AContext:
    """State of one rank for one (config, process group): buffers, peer mappings, flags."""

    def __init__(self, cfg: MoEConfig, rank: int, world_size: int, *, device: Optional[int] = None,
                 payload: str = "direct", schedule: str = "phased", combine: str = "pull",
                 chunks: Optional[int] = None, senders: int = 0,
                 timeout_ms: Optional[int] = None, group=None, connect: bool = True):
        if cfg.in_dtype != cfg.out_dtype or cfg.in_dtype not in _DTYPES:
            raise A2AError(_lib.A2A_ERR_CONFIG, f"unsupported dtypes {cfg.in_dtype}/{cfg.out_dtype}")
        self.lib = _lib.load()
        if timeout_ms is None:
            # budget of every device-side wait on a peer; ranks must reach a call within it of each other
            timeout_ms = int(os.environ.get("A2A_TIMEOUT_MS", "5000"))
        if chunks is None:
            # token chunks of the phased schedule; resolved here so that it travels in the configuration
            # fingerprint the ranks compare (a rank with another value is refused at set-up)
            chunks = int(os.environ.get("A2A_CHUNKS", "1")) if schedule == "phased" else 1
        self.cfg, self.rank, self.world_size = cfg, rank, world_size
        self.payload, self.schedule, self.combine_mode = payload, schedule, combine
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device_index = int(device)
        self.device = torch.device("cuda", self.device_index)
        self.group = group
        c = Config(rank, world_size, self.device_index, cfg.num_experts, cfg.experts_per_token,
                   cfg.hidden_dim, cfg.max_num_tokens, _DTYPES[cfg.in_dtype], _lib.PAYLOAD[payload], timeout_ms,
                   _lib.SCHEDULE[schedule], _lib.COMBINE[combine], max(1, min(4, int(chunks))), int(senders))
        self._h = C.c_void_p()
        _lib.check(self.lib.a2a_create(C.byref(self._h), C.byref(c)))
        self.num_local_experts = cfg.num_experts // world_size
        self.max_recv = cfg.max_num_tokens * world_size
        self._num_tokens = 0
        if connect and world_size > 1:
            self._connect_over_group()

    # ---- bootstrap ---------------------------------------------------------
    def export_handle(self) -> torch.Tensor:
        n = self.lib.a2a_ipc_handle_bytes()
        blob = torch.empty(n, dtype=torch.uint8)
        _lib.check(self.lib.a2a_export_handle(self._h, _ptr(blob)))
        return blob

    def open_peers(self, all_blobs: torch.Tensor) -> None:
        """Map the peers from the gathered blobs; refuses (A2A_ERR_CONFIG, with the library's
        description) a short gather or a rank whose configuration differs from ours."""
        all_blobs = all_blobs.contiguous().cpu()
        rc = self.lib.a2a_open_peers(self._h, _ptr(all_blobs), all_blobs.numel())
        if rc == _lib.A2A_ERR_CONFIG:
            raise A2AError(rc, self.lib.a2a_last_error(self._h).decode() or _lib.strerror(rc))
        _lib.check(rc)

    def _connect_over_group(self) -> None:
        """One all_gather of the handle blobs over the caller's process group, then map the peers."""
        blob = self.export_handle()
        backend = dist.get_backend(self.group)
        on_gpu = "nccl" in str(backend)
        mine = blob.to(self.device) if on_gpu else blob
        gathered = torch.empty(self.world_size * blob.numel(), dtype=torch.uint8, device=mine.device)
        dist.all_gather_into_tensor(gathered, mine, group=self.group)
        self.open_peers(gathered)
        # nobody may write into a region before its owner has finished zeroing it
        # (a2a_create synchronised), and everybody has now mapped everybody
        dist.barrier(group=self.group)

    @staticmethod
    def attach_local(ctxs: Sequence["A2AContext"]) -> None:
        """Wire up contexts that live in this process (rank r at position r)."""
        arr = (C.c_void_p * len(ctxs))(*[c._h for c in ctxs])
        for c in ctxs:
            rc = c.lib.a2a_attach_local_peers(c._h, arr)
            if rc == _lib.A2A_ERR_CONFIG:
                raise A2AError(rc, c.lib.a2a_last_error(c._h).decode() or _lib.strerror(rc))
            _lib.check(rc)

    # ---- phases ------------------------------------------------------------
    @staticmethod
    def _stream() -> C.c_void_p:
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def route(self, indices: torch.Tensor) -> None:
        assert indices.dtype == torch.int32 and indices.is_contiguous() and indices.is_cuda
        self._num_tokens = indices.shape[0]
        self._keep = [indices]
        _lib.check(self.lib.a2a_route(self._h, _ptr(indices), self._num_tokens, self._stream()))

    def dispatch_send(self, x: torch.Tensor) -> None:
        assert x.dtype == self.cfg.in_dtype and x.is_contiguous() and x.is_cuda
        self._keep.append(x)
        _lib.check(self.lib.a2a_dispatch_send(self._h, _ptr(x), self._stream()))

    def dispatch_recv(self) -> None:
        _lib.check(self.lib.a2a_dispatch_recv(self._h, self._stream()))

    def expert_placeholder(self) -> None:
        _lib.check(self.lib.a2a_expert_placeholder(self._h, self._stream()))

    def dispatch_recv_expert(self) -> None:
        _lib.check(self.lib.a2a_dispatch_recv_expert(self._h, self._stream()))

    def expert_done(self) -> None:
        _lib.check(self.lib.a2a_expert_done(self._h, self._stream()))

    def combine(self, weights: torch.Tensor, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert weights.dtype == torch.float32 and weights.is_contiguous() and weights.is_cuda
        if y is None:
            y = torch.empty(self._num_tokens, self.cfg.hidden_dim, dtype=self.cfg.out_dtype, device=self.device)
        self._keep.append(weights)
        _lib.check(self.lib.a2a_combine(self._h, _ptr(weights), _ptr(y), self._stream()))
        return y

    def _check_inputs(self, x, indices, weights, y, on_device: bool) -> int:
        """The library reads raw pointers: refuse anything whose bytes would be misread."""
        n, K, H = x.shape[0], self.cfg.experts_per_token, self.cfg.hidden_dim
        bad = None
        if x.dtype != self.cfg.in_dtype or tuple(x.shape) != (n, H):
            bad = f"x must be [{n}, {H}] {self.cfg.in_dtype}, got {tuple(x.shape)} {x.dtype}"
        elif indices.dtype != torch.int32 or tuple(indices.shape) != (n, K):
            bad = f"indices must be [{n}, {K}] int32, got {tuple(indices.shape)} {indices.dtype}"
        elif weights.dtype != torch.float32 or tuple(weights.shape) != (n, K):
            bad = f"weights must be [{n}, {K}] float32, got {tuple(weights.shape)} {weights.dtype}"
        elif y is not None and (y.dtype != self.cfg.out_dtype or tuple(y.shape) != (n, H)):
            bad = f"y must be [{n}, {H}] {self.cfg.out_dtype}, got {tuple(y.shape)} {y.dtype}"
        else:
            for name, t in (("x", x), ("indices", indices), ("weights", weights), ("y", y)):
                if t is None:
                    continue
                if not t.is_contiguous():
                    bad = f"{name} must be contiguous"
                elif on_device and (not t.is_cuda or t.device.index != self.device_index):
                    bad = f"{name} must live on cuda:{self.device_index}, got {t.device}"
                elif not on_device and t.is_cuda:
                    bad = f"{name} must be a host tensor"
        if bad:
            raise A2AError(_lib.A2A_ERR_CONFIG, bad)
        return n

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """route + dispatch + expert placeholder + combine on the current stream (device tensors)."""
        n = self._check_inputs(x, indices, weights, y, on_device=True)
        if y is None:
            y = torch.empty(n, self.cfg.hidden_dim, dtype=self.cfg.out_dtype, device=self.device)
        self._num_tokens = n
        _lib.check(self.lib.a2a_forward(self._h, _ptr(x), _ptr(indices), _ptr(weights), _ptr(y), n, self._stream()))
        return y

    def pipe_step(self, role: int, x=None, indices=None, weights=None, y=None) -> Optional[torch.Tensor]:
        """One role of the pipelined kernel as its own launch: 0 senders + routers (takes x, indices,
        weights and optionally the output tensor), 1 experts, 2 combine (returns the output).  For
        stepping several ranks on one GPU and for timing the roles apart."""
        if role == 0:
            n = self._check_inputs(x, indices, weights, y, on_device=True)
            if y is None:
                y = torch.empty(n, self.cfg.hidden_dim, dtype=self.cfg.out_dtype, device=self.device)
            self._num_tokens, self._y = n, y
            self._keep = [x, indices, weights, y]
            _lib.check(self.lib.a2a_pipe_step(self._h, 0, _ptr(x), _ptr(indices), _ptr(weights), _ptr(y), n,
                                              self._stream()))
            return None
        _lib.check(self.lib.a2a_pipe_step(self._h, role, None, None, None, None, self._num_tokens, self._stream()))
        return self._y if role == 2 else None

    def forward_host(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                     y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Same for HOST tensors (pinned for speed): copies in, runs, copies out, all asynchronous."""
        n = self._check_inputs(x, indices, weights, y, on_device=False)
        if y is None:
            y = torch.empty(n, self.cfg.hidden_dim, dtype=self.cfg.out_dtype, pin_memory=torch.cuda.is_available())
        self._num_tokens = n
        _lib.check(self.lib.a2a_forward_host(self._h, _ptr(x), _ptr(indices), _ptr(weights), _ptr(y), n,
                                             self._stream()))
        return y

    def set_fused(self, on: bool) -> None:
        """forward() as one cooperative launch (default) or as one kernel per phase."""
        _lib.check(self.lib.a2a_set_fused(self._h, 1 if on else 0))

    def barrier(self) -> None:
        _lib.check(self.lib.a2a_barrier(self._h, self._stream()))

    def link_probe(self, peer: int, nbytes: int) -> None:
        """Enqueue one peer copy of ``nbytes`` from our slab rows into ``peer``'s (measurement helper)."""
        _lib.check(self.lib.a2a_link_probe(self._h, peer, nbytes, self._stream()))

    # ---- inspection --------------------------------------------------------
    def export_dispatch(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """What ``PyTorchAllToAll.dispatch`` returns (reference.py:148); padding is zero here."""
        L, R, H = self.num_local_experts, self.max_recv, self.cfg.hidden_dim
        counts = torch.zeros(L, dtype=torch.int32, device=self.device)
        rows = torch.zeros(L, R, H, dtype=self.cfg.in_dtype, device=self.device)
        meta = torch.zeros(L, R, 5, dtype=torch.int32, device=self.device)
        _lib.check(self.lib.a2a_export_dispatch(self._h, _ptr(counts), _ptr(rows), _ptr(meta), self._stream()))
        return counts, rows, meta

    def expert_buffers(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Views (no copy) of this rank's slab rows [L, world, T_max, H] and of the cumulative row counts
        [world, 4, L] -- what a real expert kernel reads and overwrites in place between
        ``dispatch_recv`` and ``expert_done``."""
        rows, counts = C.c_void_p(), C.c_void_p()
        _lib.check(self.lib.a2a_expert_buffers(self._h, C.byref(rows), C.byref(counts)))
        L, ws, T, H = self.num_local_experts, self.world_size, self.cfg.max_num_tokens, self.cfg.hidden_dim
        return (_device_view(rows.value, (L, ws, T, H), self.cfg.in_dtype, self.device_index),
                _device_view(counts.value, (ws, 4, L), torch.int32, self.device_index))

    def route_tables(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Copies of the slot table [num_tokens, K] and per-expert send counts [E] of the last route."""
        n, K, E = self._num_tokens, self.cfg.experts_per_token, self.cfg.num_experts
        out_s = torch.empty(n, K, dtype=torch.int32, device=self.device)
        out_c = torch.empty(E, dtype=torch.int32, device=self.device)
        _lib.check(self.lib.a2a_copy_route(self._h, _ptr(out_s), _ptr(out_c), self._stream()))
        return out_s, out_c

    def status(self) -> Status:
        s = Status()
        _lib.check(self.lib.a2a_status(self._h, C.byref(s)))
        return s

    def check(self) -> None:
        """Raise if a kernel of this context has recorded an error."""
        s = self.status()
        if s.code != 0:
            raise A2AError(s.code, f"{_lib.strerror(s.code)} (rank {s.rank}, peer {s.peer}, phase {s.phase}, "
                                   f"call {s.epoch}, detail {s.detail})")

    def peek(self) -> int:
        """The recorded error code (0 = none) without any CUDA call: a read of mapped host memory."""
        return int(self.lib.a2a_status_peek(self._h))

    def raise_and_clear_if_failed(self) -> None:
        """What the plugin entry does before every call: if an earlier call recorded an error,
        read it, clear it (a recorded timeout would make every later wait give up at once) and raise."""
        if self.peek() == 0:
            return
        s = self.status()
        self.clear_status()
        raise A2AError(s.code, f"an earlier call failed: {_lib.strerror(s.code)} (rank {s.rank}, peer {s.peer}, "
                               f"phase {s.phase}, call {s.epoch}, detail {s.detail}); the status has been cleared")

    def clear_status(self) -> None:
        _lib.check(self.lib.a2a_status_clear(self._h))

    STAMPS = ("global_ns", "start", "routed", "sent", "dispatch_seen", "expert_done", "expert_seen", "combine_done")
    STAMPS_PER_BLOCK = 32  # slots 8.. : per-source / per-destination stamps of the pipelined kernel

    def trace_enable(self, on: bool = True) -> None:
        """Turn the in-kernel trace on or off (synchronises the device)."""
        _lib.check(self.lib.a2a_trace_enable(self._h, 1 if on else 0))

    def trace_read(self) -> torch.Tensor:
        """Stamps of the most recent traced launch: int64 [blocks, 32] (slots 0-7 see STAMPS; SM cycles,
        slot 0 in ns; the pipelined kernel stores its role bits in slot 2 and fills slots 8-31)."""
        buf = torch.zeros(2048, self.STAMPS_PER_BLOCK, dtype=torch.int64)
        blocks, per = C.c_int(), C.c_int()
        _lib.check(self.lib.a2a_trace_read(self._h, _ptr(buf), 2048, C.byref(blocks), C.byref(per)))
        return buf[: blocks.value]

    @property
    def launches(self) -> int:
        return int(self.lib.a2a_launch_count(self._h))

    @property
    def symmetric_bytes(self) -> int:
        return int(self.lib.a2a_symmetric_bytes(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.a2a_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _RawDeviceMemory:
    """Just enough of the CUDA array interface for torch to wrap library-owned device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _device_view(ptr: int, shape, dtype: torch.dtype, device_index: int) -> torch.Tensor:
    n = 1
    for d in shape:
        n *= d
    raw = torch.as_tensor(_RawDeviceMemory(ptr, n * torch.empty((), dtype=dtype).element_size()),
                          device=torch.device("cuda", device_index))
    return raw.view(dtype).view(*shape)


# ---------------------------------------------------------------------------
# plugin entry point
# ---------------------------------------------------------------------------
_CONTEXTS: Dict[tuple, A2AContext] = {}
DEFAULT_PAYLOAD = "dedup"  # one wire row per (token, destination rank): least NVLink traffic, same results
# "auto": the pipelined one-launch kernel where the configuration allows it (DEDUP / FP8 payload, shared-memory
# limits), else the phased one.  The decision depends on the configuration only, so every rank takes the same.
DEFAULT_SCHEDULE = os.environ.get("A2A_SCHEDULE", "auto")
DEFAULT_COMBINE = os.environ.get("A2A_COMBINE", "push")  # used with the pipelined schedule; phased is always pull


def _context_for(cfg: MoEConfig, rank: int, world_size: int, device_index: int, payload: str,
                 schedule: str, combine: str) -> A2AContext:
    key = (cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens, cfg.in_dtype,
           rank, world_size, device_index, payload, schedule, combine)
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        # first call with this shape: collective set-up (every rank gets here in the same call)
        ctx = None
        if schedule in ("auto", "pipelined") and (payload in ("dedup", "fp8") or schedule == "pipelined"):
            try:
                ctx = A2AContext(cfg, rank, world_size, device=device_index, payload=payload,
                                 schedule="pipelined", combine=combine)
            except A2AError as e:
                if schedule == "pipelined" or e.code != _lib.A2A_ERR_CONFIG:
                    raise
        if ctx is None:
            ctx = A2AContext(cfg, rank, world_size, device=device_index, payload=payload)
        _CONTEXTS[key] = ctx
    return ctx


def custom_kernel(data: input_t, payload: Optional[str] = None, schedule: Optional[str] = None,
                  combine: Optional[str] = None) -> output_t:
    """dispatch -> expert placeholder -> combine for this rank (task.py:8-9).

    Device tensors in ``rank_data`` run on the current CUDA stream and return a
    device tensor without synchronising.  Host tensors take the host entry point
    (copies inside) and return a pinned host tensor after a stream synchronise.
    The inputs are not modified.  Errors a kernel records (a peer that never
    arrived, an expert index out of range) surface as ``A2AError`` at the START
    of the next call on the same context -- the check reads one word of host
    memory, so it costs nothing -- and the status is cleared so that the
    context can be used again; call ``A2AContext.check()`` after a synchronise
    to see them earlier.
    """
    cfg, rank_data, rank, world_size = data
    x, idx, w = rank_data.x, rank_data.indices, rank_data.weights
    payload = payload or DEFAULT_PAYLOAD
    schedule = schedule or DEFAULT_SCHEDULE
    combine = combine or DEFAULT_COMBINE
    device_index = x.device.index if x.is_cuda else torch.cuda.current_device()
    ctx = _context_for(cfg, rank, world_size, device_index, payload, schedule, combine)
    ctx.raise_and_clear_if_failed()
    if idx.dtype != torch.int32:
        idx = idx.to(torch.int32)
    if w.dtype != torch.float32:
        w = w.to(torch.float32)
    if x.is_cuda:
        return ctx.forward(x.contiguous(), idx.contiguous(), w.contiguous())
    y = ctx.forward_host(x.contiguous(), idx.contiguous(), w.contiguous())
    torch.cuda.current_stream().synchronize()
    return y


def check_implementation(data: input_t, output: output_t, reference_output: Optional[torch.Tensor] = None,
                         rtol: float = 1e-2, atol: float = 5e-3):
    """The task's checker (reference.py:275-283): ``(ok, message)`` for one rank's ``output``.

    The reference computes its expectation by running ``ref_kernel(data)`` -- a collective
    call of its PyTorch path.  This package ships no second implementation of the path, so
    the expectation is passed in: a harness computes it with whatever reference it trusts
    (the task's own ``ref_kernel``) and hands it over.  The comparison is the reference's:
    same device, then ``allclose`` with the task's tolerances.
    """
    if reference_output is None:
        raise ValueError("check_implementation needs reference_output (this package has no reference path)")
    if output.device != reference_output.device:
        return False, f"Output device mismatch: {output.device} != {reference_output.device}"
    if output.shape != reference_output.shape or output.dtype != reference_output.dtype:
        return False, (f"Output shape/dtype mismatch: {tuple(output.shape)} {output.dtype} != "
                       f"{tuple(reference_output.shape)} {reference_output.dtype}")
    res = torch.allclose(output, reference_output, rtol=rtol, atol=atol)
    if not res:
        diff = (output.float() - reference_output.float()).abs()
        return False, f"mismatch found! custom implementation doesn't match reference: max |diff| {float(diff.max()):.4g}"
    return True, ""


def release_contexts(barrier: bool = True) -> None:
    """Tear down every cached context (peers must have stopped touching our memory first)."""
    if not _CONTEXTS:
        return
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if barrier and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    for ctx in list(_CONTEXTS.values()):
        ctx.close()
    _CONTEXTS.clear()


# The task harness creates and destroys the process group per test case
# (my_eval.py:64-85), possibly on another GPU each time, so peer mappings must
# die with the group.  Like the reference (submission_v9.py:952-973) we hook
# destroy_process_group; set-up needs no hook because it is lazy.
_original_destroy = dist.destroy_process_group


def _destroy_with_release(*args, **kwargs):
    error = None
    try:
        release_contexts(barrier=True)
    except Exception as e:  # noqa: BLE001 - the group must still be destroyed; re-raised below
        error = e
    _original_destroy(*args, **kwargs)
    if error is not None:
        raise error


def install_process_group_hooks() -> None:
    if dist.destroy_process_group is not _destroy_with_release:
        dist.destroy_process_group = _destroy_with_release


install_process_group_hooks()
