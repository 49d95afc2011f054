"""Host-side mirror of the reference operator `mla_bwd_cuda.mla_bwd` over the C-ABI library.

Reference surface: `mla_bwd(q, kv, dO, lse, O, indices) -> (dQ, dKV)` (`mla_bwd/mla_bwd.cu:972-1063`,
called positionally by `mla_bwd/test_mla_bwd.py:103,140`).  Same positional order and the same
checks / error behaviour (`RuntimeError` for shape, dtype, device and contiguity problems); the
trailing keyword arguments are additions.  torch is used only for device memory and the current
stream; all arithmetic happens in the hand-written CUDA kernels behind `include/smla_bwd.h`.
There is no CPU or eager fallback: if the library is missing and cannot be built, import fails.
"""
from __future__ import annotations

import ctypes
import math
import os
import threading
from typing import Optional, Tuple

import torch

from . import build as _build

D_QK = 576
D_V = 512
NO_CAUSAL = -(2 ** 31)

STAGE_ZERO, STAGE_DELTA, STAGE_RECOMPUTE, STAGE_DKV, STAGE_DQ = 1, 2, 4, 8, 16
STAGE_ALL = 31


class _Params(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("kv", ctypes.c_void_p), ("dO", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("O", ctypes.c_void_p), ("indices", ctypes.c_void_p), ("dQ", ctypes.c_void_p), ("dKV", ctypes.c_void_p),
        ("s_q", ctypes.c_int32), ("s_kv", ctypes.c_int32), ("h_q", ctypes.c_int32), ("topk", ctypes.c_int32),
        ("sm_scale", ctypes.c_float), ("q_start_index_s", ctypes.c_int32), ("lse_is_base2", ctypes.c_int32),
        ("query_meta", ctypes.c_void_p),
    ]


class _FwdParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("kv", ctypes.c_void_p), ("indices", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("s_q", ctypes.c_int32), ("s_kv", ctypes.c_int32), ("h_q", ctypes.c_int32), ("topk", ctypes.c_int32),
        ("sm_scale", ctypes.c_float), ("q_start_index_s", ctypes.c_int32), ("lse_is_base2", ctypes.c_int32),
        ("query_meta", ctypes.c_void_p),
    ]


class _DetParams(ctypes.Structure):
    _fields_ = [("row_ptr", ctypes.c_void_p), ("entries", ctypes.c_void_p), ("staging", ctypes.c_void_p),
                ("staging_bytes", ctypes.c_size_t)]


class WorkspaceLayout(ctypes.Structure):
    _fields_ = [
        ("err_offset", ctypes.c_size_t), ("delta_offset", ctypes.c_size_t), ("s_offset", ctypes.c_size_t),
        ("ds_offset", ctypes.c_size_t), ("q_chunk", ctypes.c_int32), ("topk_pad", ctypes.c_int32),
        ("h_pad", ctypes.c_int32), ("total_bytes", ctypes.c_size_t),
    ]


def scratch_matrices(ws, lay):
    """The bf16 S and dS the recompute stage left in a workspace, as [q_chunk, topk_pad, h_pad] tensors.

    In the workspace each query's matrix is stored head-block-major, [h_pad/8][topk_pad][8 heads] (what the
    recompute kernel can write in whole cache lines and the later kernels fetch with one TMA box); this undoes
    that for stage-by-stage checks."""
    n = lay.q_chunk * lay.topk_pad * lay.h_pad
    out = []
    for off in (lay.s_offset, lay.ds_offset):
        m = ws.buf[off: off + 2 * n].view(torch.bfloat16).view(lay.q_chunk, lay.h_pad // 8, lay.topk_pad, 8)
        out.append(m.permute(0, 2, 1, 3).reshape(lay.q_chunk, lay.topk_pad, lay.h_pad))
    return out[0], out[1]


_lib = None
_lib_lock = threading.Lock()


def load_library() -> ctypes.CDLL:
    """Load (building first if the sources are newer) the C-ABI shared library."""
    global _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        if _build.needs_build():
            try:
                _build.build()
            except Exception as e:  # prebuilt library on a box without nvcc is fine; none at all is not
                if not os.path.exists(path):
                    raise RuntimeError(f"sparse MLA CUDA library is missing and could not be built: {e}") from e
        lib = ctypes.CDLL(path)
        lib.smla_bwd_workspace_size.restype = ctypes.c_size_t
        lib.smla_bwd_workspace_size.argtypes = [ctypes.POINTER(_Params), ctypes.c_size_t]
        lib.smla_bwd_run.restype = ctypes.c_int
        lib.smla_bwd_run.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.smla_bwd_run_stages.restype = ctypes.c_int
        lib.smla_bwd_run_stages.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                            ctypes.c_int]
        lib.smla_bwd_delta.restype = ctypes.c_int
        lib.smla_bwd_delta.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                       ctypes.c_int32, ctypes.c_void_p]
        lib.smla_bwd_get_workspace_layout.restype = ctypes.c_int
        lib.smla_bwd_get_workspace_layout.argtypes = [ctypes.POINTER(_Params), ctypes.c_size_t,
                                                      ctypes.POINTER(WorkspaceLayout)]
        lib.smla_bwd_status.restype = ctypes.c_int
        lib.smla_bwd_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.smla_bwd_run_noalloc.restype = ctypes.c_int
        lib.smla_bwd_run_noalloc.argtypes = [ctypes.POINTER(_Params), ctypes.c_void_p]
        lib.smla_bwd_noalloc_capacity.restype = ctypes.c_size_t
        lib.smla_bwd_noalloc_status.restype = ctypes.c_int
        lib.smla_bwd_noalloc_status.argtypes = [ctypes.c_void_p]
        lib.smla_fwd_workspace_size.restype = ctypes.c_size_t
        lib.smla_fwd_workspace_size.argtypes = [ctypes.POINTER(_FwdParams), ctypes.c_size_t]
        lib.smla_fwd_run.restype = ctypes.c_int
        lib.smla_fwd_run.argtypes = [ctypes.POINTER(_FwdParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.smla_bwd_last_launch_count.restype = ctypes.c_int
        lib.smla_index_inverse_workspace_size.restype = ctypes.c_size_t
        lib.smla_index_inverse_workspace_size.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
        lib.smla_index_inverse.restype = ctypes.c_int
        lib.smla_index_inverse.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                           ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_size_t, ctypes.c_void_p]
        lib.smla_bwd_workspace_init.restype = ctypes.c_int
        lib.smla_bwd_workspace_init.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.smla_bwd_last_device_code.restype = ctypes.c_int
        lib.smla_bwd_set_schedule.restype = ctypes.c_int
        lib.smla_bwd_set_schedule.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.smla_bwd_get_schedule.restype = None
        lib.smla_bwd_get_schedule.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        lib.smla_debug_set_wait_limit_cycles.restype = ctypes.c_int
        lib.smla_debug_set_wait_limit_cycles.argtypes = [ctypes.c_longlong]
        lib.smla_selftest_wait_timeout.restype = ctypes.c_int
        lib.smla_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                                                   ctypes.c_void_p]
        lib.smla_bwd_run_deterministic.restype = ctypes.c_int
        lib.smla_bwd_run_deterministic.argtypes = [ctypes.POINTER(_Params), ctypes.POINTER(_DetParams), ctypes.c_void_p,
                                                   ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int]
        lib.smla_bwd_staging_bytes_per_query.restype = ctypes.c_size_t
        lib.smla_bwd_staging_bytes_per_query.argtypes = [ctypes.POINTER(_Params)]
        lib.smla_dkv_pull_reduce.restype = ctypes.c_int
        lib.smla_dkv_pull_reduce.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                             ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
        lib.smla_dkv_multimem_reduce.restype = ctypes.c_int
        lib.smla_dkv_multimem_reduce.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                                 ctypes.c_int32, ctypes.c_void_p]
        lib.smla_clock_probe.restype = ctypes.c_int
        lib.smla_clock_probe.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.smla_reduction_rate_probe.restype = ctypes.c_int
        lib.smla_reduction_rate_probe.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                  ctypes.c_void_p]
        lib.smla_bwd_status_string = lib.smla_status_string
        lib.smla_status_string.restype = ctypes.c_char_p
        lib.smla_status_string.argtypes = [ctypes.c_int]
        _lib = lib
        return lib


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _raise_status(lib, status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what}: {lib.smla_status_string(status).decode()} (status {status})")


class Workspace:
    """Device scratch owned by the caller (delta, bf16 S / dS, error word); reusable across calls.

    The first 256 bytes hold the device error word and start at zero; the kernels only ever set it, and
    `device_status` clears it after reporting."""

    def __init__(self, nbytes: int, device):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf[:256].zero_()
        self.nbytes = nbytes

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()


# Workspaces handed out when the caller passes none, one per (device, stream) so that calls queued on different
# streams do not share scratch; kept (and grown when a larger problem comes) instead of allocating gigabytes per call.
_ws_cache = {}
_ws_cache_lock = threading.Lock()


def _cached_workspace(need: int, device: torch.device) -> Workspace:
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    with _ws_cache_lock:
        ws = _ws_cache.get(key)
        if ws is None or ws.nbytes < need:
            _ws_cache.pop(key, None)
            ws = None                       # let the smaller one go before the larger one is allocated
            ws = Workspace(need, device)
            _ws_cache[key] = ws
        return ws


_buf_cache = {}


def _cached_buffer(kind: str, need: int, device: torch.device) -> torch.Tensor:
    """A byte buffer kept per (kind, device, stream) and grown on demand, like the workspaces."""
    key = (kind, device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    with _ws_cache_lock:
        buf = _buf_cache.get(key)
        if buf is None or buf.numel() < need:
            _buf_cache.pop(key, None)
            buf = None
            buf = torch.empty(need, dtype=torch.uint8, device=device)
            _buf_cache[key] = buf
        return buf


def release_cached_workspaces() -> None:
    """Drop the workspaces and staging buffers kept for calls that pass none (they are re-created on demand)."""
    with _ws_cache_lock:
        _ws_cache.clear()
        _buf_cache.clear()


def _make_params(q, kv2, dO, lse, O, idx2, dQ, dKV2, sm_scale, q_start_index_s, lse_is_base2,
                 query_meta=None) -> _Params:
    return _Params(
        q.data_ptr(), kv2.data_ptr(), dO.data_ptr(), lse.data_ptr(), O.data_ptr(), idx2.data_ptr(),
        dQ.data_ptr(), dKV2.data_ptr(),
        q.shape[0], kv2.shape[0], q.shape[1], idx2.shape[1],
        float(sm_scale) if sm_scale is not None else 0.0,
        NO_CAUSAL if q_start_index_s is None else int(q_start_index_s),
        1 if lse_is_base2 else 0,
        query_meta.data_ptr() if query_meta is not None else None,
    )


def _check_query_meta(query_meta, q) -> None:
    if query_meta is None:
        return
    _check(isinstance(query_meta, torch.Tensor) and query_meta.is_cuda and query_meta.device == q.device
           and query_meta.dtype == torch.int32 and query_meta.is_contiguous()
           and tuple(query_meta.shape) == (q.shape[0], 4) and query_meta.data_ptr() % 16 == 0,
           "query_meta must be a contiguous int32 CUDA tensor [s_q, 4] on q's device")


def _check_out(t, like_shape_numel, dtype, device, name) -> None:
    _check(isinstance(t, torch.Tensor) and t.is_cuda and t.device == device and t.dtype == dtype and t.is_contiguous()
           and t.numel() == like_shape_numel, f"{name} must be a contiguous {dtype} CUDA tensor of {like_shape_numel} elements on {device}")


def _validate(q, kv, dO, lse, O, indices):
    """The reference's TORCH_CHECKs (`mla_bwd/mla_bwd.cu:975-1015`), widened to h_q in {8..128} and 3-D kv/indices."""
    for name, t in (("q", q), ("kv", kv), ("dO", dO), ("lse", lse), ("O", O), ("indices", indices)):
        _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
        _check(t.is_contiguous(), f"{name} must be contiguous")
        _check(t.device == q.device, f"{name} must be on the same device as q")
    _check(q.dtype == torch.bfloat16, "q must be bfloat16")
    _check(kv.dtype == torch.bfloat16, "kv must be bfloat16")
    _check(dO.dtype == torch.bfloat16, "dO must be bfloat16")
    _check(O.dtype == torch.bfloat16, "O must be bfloat16")
    _check(lse.dtype == torch.float32, "lse must be float32")
    _check(indices.dtype == torch.int32, "indices must be int32")
    _check(q.dim() == 3, "q must have shape [s_q, h_q, 576]")
    _check(kv.dim() in (2, 3), "kv must have shape [s_kv, 576] or [s_kv, 1, 576]")
    _check(indices.dim() in (2, 3), "indices must have shape [s_q, topk] or [s_q, 1, topk]")
    if kv.dim() == 3:
        _check(kv.shape[1] == 1, "only h_kv = 1 is supported")
    if indices.dim() == 3:
        _check(indices.shape[1] == 1, "only h_kv = 1 is supported")
    s_q, h_q, d_qk = q.shape
    _check(d_qk == D_QK, f"q last dim must be {D_QK}")
    _check(kv.shape[-1] == D_QK, f"kv last dim must be {D_QK}")
    _check(0 < h_q <= 128 and h_q % 8 == 0, f"h_q must be a multiple of 8 in [8, 128], got {h_q}")
    _check(tuple(dO.shape) == (s_q, h_q, D_V), f"dO must have shape [{s_q}, {h_q}, {D_V}]")
    _check(tuple(O.shape) == (s_q, h_q, D_V), f"O must have shape [{s_q}, {h_q}, {D_V}]")
    _check(tuple(lse.shape) == (s_q, h_q), f"lse must have shape [{s_q}, {h_q}]")
    _check(indices.shape[0] == s_q, "indices first dim must equal s_q")
    topk = indices.shape[-1]
    _check(topk > 0, "topk must be positive")


def mla_bwd(
    q: torch.Tensor, kv: torch.Tensor, dO: torch.Tensor, lse: torch.Tensor, O: torch.Tensor, indices: torch.Tensor,
    sm_scale: Optional[float] = None,
    q_start_index_s: Optional[int] = 0,
    lse_is_base2: bool = True,
    out_dkv: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    workspace: Optional[Workspace] = None,
    workspace_budget: int = 0,
    check_device_status: bool = False,
    out_dq: Optional[torch.Tensor] = None,
    query_meta: Optional[torch.Tensor] = None,
    deterministic: bool = False,
    staging_budget: int = 2 << 30,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse MLA attention backward.  Returns (dQ bf16 [s_q,h_q,576], dKV fp32 shaped like kv).

    Positional arguments and defaults are the reference operator's: base-2 `lse`, sm_scale =
    1/sqrt(576), and the causal rule "slot valid only if idx <= query row" (`q_start_index_s=0`,
    `mla_bwd/mla_bwd.cu:122,772`).  Pass `q_start_index_s=None` to keep only the range check.
    `out_dkv` + `accumulate=True` add into an existing fp32 buffer (partial dKV of a query shard);
    `out_dq` receives dQ in place.  `query_meta` (int32 [s_q, 4] on the device: first kv row and number of
    kv rows of the query's sequence, position for the causal rule, top-k slots in use) lets one call cover
    packed sequences; see `query_meta_for`.  Without `workspace` the scratch comes from a cache kept per
    (device, stream).  `deterministic=True` makes dKV reproducible bit for bit (dQ always is): the index inverse of the
    sparse pattern is built (`index_inverse`), every slot's contribution goes to a staging buffer of at most about
    `staging_budget` bytes and is added per kv row in a fixed order - slower (one extra write and read of 2304
    bytes per slot), for runs that must repeat exactly.  The call enqueues on the current stream and does not
    synchronise unless `check_device_status=True`, which also raises if a kernel reported a timed-out wait.
    """
    _validate(q, kv, dO, lse, O, indices)
    _check_query_meta(query_meta, q)
    lib = load_library()
    kv2 = kv.reshape(kv.shape[0], D_QK)
    idx2 = indices.reshape(indices.shape[0], indices.shape[-1])
    with torch.cuda.device(q.device):
        if out_dq is None:
            dQ = torch.empty_like(q)
        else:
            _check_out(out_dq, q.numel(), torch.bfloat16, q.device, "out_dq")
            dQ = out_dq
        if out_dkv is None:
            dKV = torch.empty(kv.shape, dtype=torch.float32, device=q.device)
            _check(not accumulate, "accumulate=True needs out_dkv")
        else:
            _check_out(out_dkv, kv.numel(), torch.float32, q.device, "out_dkv")
            dKV = out_dkv
        params = _make_params(q, kv2, dO, lse, O, idx2, dQ, dKV, sm_scale, q_start_index_s, lse_is_base2, query_meta)
        if workspace is None:
            need = lib.smla_bwd_workspace_size(ctypes.byref(params), workspace_budget)
            _check(need > 0, "unsupported shapes for the sparse MLA backward")
            # a budget asks for a particular size: do not serve it from a (possibly larger) cached one
            workspace = Workspace(need, q.device) if workspace_budget else _cached_workspace(need, q.device)
        stream = torch.cuda.current_stream().cuda_stream
        stages = STAGE_ALL & ~STAGE_ZERO if accumulate else STAGE_ALL
        if deterministic:
            _check(query_meta is None, "deterministic=True handles one sequence per call (no query_meta)")
            row_ptr, entries = index_inverse(idx2, kv2.shape[0], q_start_index_s)
            per_q = lib.smla_bwd_staging_bytes_per_query(ctypes.byref(params))
            n_stage = max(1, min(q.shape[0], max(int(staging_budget), per_q) // per_q))
            staging = _cached_buffer("staging", n_stage * per_q, q.device)
            det = _DetParams(row_ptr.data_ptr(), entries.data_ptr(), staging.data_ptr(), staging.numel())
            st = lib.smla_bwd_run_deterministic(ctypes.byref(params), ctypes.byref(det), workspace.ptr, workspace.nbytes,
                                                stream, stages)
            for t in (row_ptr, entries):
                t.record_stream(torch.cuda.current_stream())
        else:
            st = lib.smla_bwd_run_stages(ctypes.byref(params), workspace.ptr, workspace.nbytes, stream, stages)
        _raise_status(lib, st, "smla_bwd_run")
        if check_device_status:
            _raise_status(lib, lib.smla_bwd_status(workspace.ptr, stream), "smla_bwd device status")
    return dQ, dKV


def query_meta_for(seq_q_start, seq_q_len, seq_kv_start, seq_kv_len, device, q_start_index_s: Optional[int] = 0,
                   topk: int = 0, topk_length: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-query table for packed sequences: int32 [T_q, 4] = (first kv row of the query's sequence, kv rows of
    that sequence, position for the causal rule = q_start_index_s + row inside the sequence, top-k slots in use).

    `seq_*` are host integer sequences (one entry per sequence, queries and kv rows packed in that order);
    `topk_length` ([T_q], optional) limits the slots in use per query, the per-query field of the reference's
    richer parameter block (`dq_test/dq_phase_capture.cuh:107-109`)."""
    n_seq = len(seq_q_len)
    lens = torch.tensor(list(seq_q_len), dtype=torch.int64)
    seq_of_q = torch.repeat_interleave(torch.arange(n_seq), lens)
    t_q = int(lens.sum().item())
    row_in_seq = torch.arange(t_q) - torch.tensor(list(seq_q_start), dtype=torch.int64)[seq_of_q]
    meta = torch.empty(t_q, 4, dtype=torch.int32)
    meta[:, 0] = torch.tensor(list(seq_kv_start), dtype=torch.int32)[seq_of_q]
    meta[:, 1] = torch.tensor(list(seq_kv_len), dtype=torch.int32)[seq_of_q]
    meta[:, 2] = (row_in_seq + (q_start_index_s or 0)).to(torch.int32)
    meta[:, 3] = topk
    meta = meta.to(device)
    if topk_length is not None:
        _check(not topk_length.is_floating_point() and topk_length.numel() == t_q, "topk_length must be an integer tensor with one entry per query")
        meta[:, 3] = topk_length.reshape(-1).to(device=device, dtype=torch.int32).clamp(0, topk)
    return meta.contiguous()


def mla_bwd_batched(q, kv, dO, lse, O, indices, topk_length: Optional[torch.Tensor] = None,
                    q_start_index_s: Optional[int] = 0, **kwargs):
    """Backward for a batch of independent sequences of equal shape, so that callers stop looping themselves.

    q / dO / O [B, s_q, h_q, d], kv [B, s_kv, 576] (or [B, s_kv, 1, 576]), lse [B, s_q, h_q], indices [B, s_q, topk]
    with values relative to the own sequence's kv; `topk_length` [B, s_q] (optional) limits the slots in use per query.
    The batch runs as ONE chain of kernels over all B * s_q queries (a per-query table tells the kernels which kv rows
    a query may touch), writing dQ and dKV in place.  Returns (dQ [B, s_q, h_q, 576] bf16, dKV fp32 shaped like kv).
    Keyword arguments as for `mla_bwd` (without out_dkv / out_dq).
    """
    _check(q.dim() == 4 and kv.dim() in (3, 4) and indices.dim() == 3, "batched tensors need a leading batch dimension")
    B, s_q = q.shape[0], q.shape[1]
    s_kv = kv.shape[1]
    _check(all(t.shape[0] == B for t in (kv, dO, lse, O, indices)), "batch sizes differ")
    for k in ("out_dkv", "accumulate", "out_dq", "query_meta"):
        _check(k not in kwargs, "mla_bwd_batched allocates its outputs and builds its own query table")
    meta = query_meta_for([b * s_q for b in range(B)], [s_q] * B, [b * s_kv for b in range(B)], [s_kv] * B, q.device,
                          q_start_index_s, indices.shape[-1], topk_length)
    dQ = torch.empty_like(q)
    dKV = torch.empty(kv.shape, dtype=torch.float32, device=q.device)
    mla_bwd(q.reshape(B * s_q, *q.shape[2:]), kv.reshape(B * s_kv, D_QK), dO.reshape(B * s_q, *dO.shape[2:]),
            lse.reshape(B * s_q, -1), O.reshape(B * s_q, *O.shape[2:]), indices.reshape(B * s_q, -1),
            q_start_index_s=q_start_index_s, out_dq=dQ, out_dkv=dKV, query_meta=meta, **kwargs)
    return dQ, dKV


def mla_bwd_varlen(q, kv, dO, lse, O, indices, cu_seqlens_q, cu_seqlens_kv, topk_length: Optional[torch.Tensor] = None,
                   q_start_index_s: Optional[int] = 0, **kwargs):
    """Backward for sequences of different lengths packed along the first dimension.

    q / dO / O [T_q, h_q, d], lse [T_q, h_q], indices [T_q, topk], kv [T_kv, 576]; sequence i owns query rows
    cu_seqlens_q[i]:cu_seqlens_q[i+1] and kv rows cu_seqlens_kv[i]:cu_seqlens_kv[i+1] (host integer sequences or CPU
    tensors, as in the usual varlen attention interfaces).  Index values are relative to the own sequence's first kv
    row; `q_start_index_s` applies to every sequence from its own first query.  All sequences run as ONE chain of
    kernels.  Returns (dQ [T_q, h_q, 576] bf16, dKV [T_kv, 576] fp32).  Empty sequences are allowed.
    """
    cq = [int(v) for v in cu_seqlens_q]
    ck = [int(v) for v in cu_seqlens_kv]
    _check(len(cq) == len(ck) and len(cq) >= 2 and cq[0] == 0 and ck[0] == 0, "cu_seqlens must start at 0 and match in length")
    _check(cq[-1] == q.shape[0] and ck[-1] == kv.shape[0], "cu_seqlens do not cover q / kv")
    _check(all(a <= b for a, b in zip(cq, cq[1:])) and all(a <= b for a, b in zip(ck, ck[1:])), "cu_seqlens must not decrease")
    _check(all(q1 == q0 or k1 > k0 for q0, q1, k0, k1 in zip(cq, cq[1:], ck, ck[1:])), "a sequence with queries needs kv rows")
    for k in ("out_dkv", "accumulate", "out_dq", "query_meta"):
        _check(k not in kwargs, "mla_bwd_varlen allocates its outputs and builds its own query table")
    if q.shape[0] == 0:
        return torch.empty_like(q), torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
    meta = query_meta_for(cq[:-1], [b - a for a, b in zip(cq, cq[1:])], ck[:-1], [b - a for a, b in zip(ck, ck[1:])],
                          q.device, q_start_index_s, indices.shape[-1], topk_length)
    return mla_bwd(q, kv, dO, lse, O, indices, q_start_index_s=q_start_index_s, query_meta=meta, **kwargs)


def mla_fwd(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: Optional[float] = None,
            q_start_index_s: Optional[int] = 0, lse_is_base2: bool = True, workspace: Optional[Workspace] = None,
            workspace_budget: int = 0, check_device_status: bool = False,
            query_meta: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse MLA attention forward for the same top-k indices: returns (o bf16 [s_q,h_q,512], lse fp32 [s_q,h_q]).

    The reference has no forward operator; its tests make o / lse with fp32 torch code
    (`dq_test/test_dq_phase.py:53-59`).  Defaults mirror `mla_bwd` (causal rule with query start 0, base-2
    lse) so that `mla_bwd(q, kv, dO, lse, o, indices)` can consume the outputs directly.
    """
    for name, t in (("q", q), ("kv", kv), ("indices", indices)):
        _check(isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous CUDA tensor")
    _check(q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and indices.dtype == torch.int32, "dtypes: bf16, bf16, int32")
    _check(q.dim() == 3 and q.shape[2] == D_QK and kv.shape[-1] == D_QK, f"q [s_q,h_q,{D_QK}], kv [s_kv,{D_QK}]")
    _check(kv.dim() == 2 or (kv.dim() == 3 and kv.shape[1] == 1), "kv must be [s_kv,576] or [s_kv,1,576]")
    _check(indices.shape[0] == q.shape[0] and (indices.dim() == 2 or (indices.dim() == 3 and indices.shape[1] == 1)),
           "indices must be [s_q,topk] or [s_q,1,topk]")
    s_q, h_q, _ = q.shape
    _check(0 < h_q <= 128 and h_q % 8 == 0, f"h_q must be a multiple of 8 in [8, 128], got {h_q}")
    _check_query_meta(query_meta, q)
    lib = load_library()
    with torch.cuda.device(q.device):
        o = torch.empty(s_q, h_q, D_V, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(s_q, h_q, dtype=torch.float32, device=q.device)
        params = _FwdParams(q.data_ptr(), kv.data_ptr(), indices.data_ptr(), o.data_ptr(), lse.data_ptr(),
                            s_q, kv.shape[0], h_q, indices.shape[-1],
                            float(sm_scale) if sm_scale is not None else 0.0,
                            NO_CAUSAL if q_start_index_s is None else int(q_start_index_s), 1 if lse_is_base2 else 0,
                            query_meta.data_ptr() if query_meta is not None else None)
        if workspace is None:
            need = lib.smla_fwd_workspace_size(ctypes.byref(params), workspace_budget)
            _check(need > 0, "unsupported shapes for the sparse MLA forward")
            workspace = Workspace(need, q.device)
        stream = torch.cuda.current_stream().cuda_stream
        _raise_status(lib, lib.smla_fwd_run(ctypes.byref(params), workspace.ptr, workspace.nbytes, stream), "smla_fwd_run")
        if check_device_status:
            _raise_status(lib, lib.smla_bwd_status(workspace.ptr, stream), "smla_fwd device status")
    return o, lse


class SparseMLAFunction(torch.autograd.Function):
    """o = sparse_mla(q, kv, indices): forward and backward both in the hand-written kernels."""

    @staticmethod
    def forward(ctx, q, kv, indices, sm_scale, q_start_index_s):
        o, lse = mla_fwd(q, kv, indices, sm_scale=sm_scale, q_start_index_s=q_start_index_s)
        ctx.save_for_backward(q, kv, indices, o, lse)
        ctx.sm_scale, ctx.q_start = sm_scale, q_start_index_s
        return o

    @staticmethod
    def backward(ctx, dO):
        q, kv, indices, o, lse = ctx.saved_tensors
        dq, dkv = mla_bwd(q, kv, dO.contiguous(), lse, o, indices, sm_scale=ctx.sm_scale, q_start_index_s=ctx.q_start)
        return dq, dkv.to(kv.dtype), None, None, None


def sparse_mla(q, kv, indices, sm_scale: Optional[float] = None, q_start_index_s: Optional[int] = 0):
    """Differentiable sparse MLA attention (bf16 in, bf16 out; gradients for q and kv)."""
    return SparseMLAFunction.apply(q, kv, indices, sm_scale, q_start_index_s)


def index_inverse(indices: torch.Tensor, s_kv: int, q_start_index_s: Optional[int] = None):
    """CSR by kv row of the valid slots of `indices` [s_q, topk] (or [s_q, 1, topk]) int32 on a CUDA device.

    Returns (row_ptr [s_kv + 1] int32, entries [s_q * topk] int32): `entries[row_ptr[r]:row_ptr[r + 1]]` are the flat
    slot ids `q * topk + slot` that chose kv row r, ascending; behind `row_ptr[s_kv]` follow the unused slots in
    ascending flat order.  The order is fixed, so two calls agree bit for bit.  Validity as in the backward
    (`mla_bwd/mla_bwd.cu:765-789`): `0 <= idx < s_kv`, and `idx <= q_start_index_s + q` unless that is None."""
    _check(indices.is_cuda and indices.dtype == torch.int32 and indices.is_contiguous(), "indices must be a contiguous CUDA int32 tensor")
    _check(indices.dim() in (2, 3) and (indices.dim() == 2 or indices.shape[1] == 1), "indices must be [s_q, topk] or [s_q, 1, topk]")
    s_q, topk = indices.shape[0], indices.shape[-1]
    lib = load_library()
    need = lib.smla_index_inverse_workspace_size(s_q, topk, s_kv)
    _check(need > 0, "unsupported shape (s_kv and topk positive, s_q * topk below 2^31)")
    with torch.cuda.device(indices.device):
        ws = torch.empty(need, dtype=torch.uint8, device=indices.device)
        row_ptr = torch.empty(s_kv + 1, dtype=torch.int32, device=indices.device)
        entries = torch.empty(s_q * topk, dtype=torch.int32, device=indices.device)
        st = lib.smla_index_inverse(indices.data_ptr(), s_q, topk, s_kv,
                                    NO_CAUSAL if q_start_index_s is None else int(q_start_index_s),
                                    row_ptr.data_ptr(), entries.data_ptr(), ws.data_ptr(), need,
                                    torch.cuda.current_stream().cuda_stream)
    _raise_status(lib, st, "smla_index_inverse")
    return row_ptr, entries


def mla_bwd_noalloc(q, kv, dO, lse, O, indices, dQ, dKV, sm_scale: Optional[float] = None,
                    q_start_index_s: Optional[int] = 0, lse_is_base2: bool = True) -> None:
    """Backward into caller-owned `dQ` / `dKV` using the library's built-in scratch: nothing is allocated,
    neither here nor in the library.  For callers that must not touch the device allocator (see
    `smla_bwd_run_noalloc` in include/smla_bwd.h for who they are and for the size limit).  Calls on one device
    must not overlap: they share the scratch."""
    _validate(q, kv, dO, lse, O, indices)
    _check_out(dQ, q.numel(), torch.bfloat16, q.device, "dQ")
    _check_out(dKV, kv.numel(), torch.float32, q.device, "dKV")
    lib = load_library()
    params = _make_params(q, kv.view(kv.shape[0], D_QK), dO, lse, O, indices.view(indices.shape[0], indices.shape[-1]),
                          dQ, dKV, sm_scale, q_start_index_s, lse_is_base2)
    with torch.cuda.device(q.device):
        st = lib.smla_bwd_run_noalloc(ctypes.byref(params), torch.cuda.current_stream().cuda_stream)
    _raise_status(lib, st, "smla_bwd_run_noalloc")


def run_stages(q, kv, dO, lse, O, indices, dQ, dKV, workspace: Workspace, stages: int, sm_scale=None,
               q_start_index_s: Optional[int] = 0, lse_is_base2: bool = True) -> WorkspaceLayout:
    """Run selected kernels (bit mask of STAGE_*) on caller-owned outputs; returns the workspace layout.
    For stage-by-stage tests and for profiling one kernel at a time."""
    _validate(q, kv, dO, lse, O, indices)
    lib = load_library()
    kv2 = kv.reshape(kv.shape[0], D_QK)
    idx2 = indices.reshape(indices.shape[0], indices.shape[-1])
    params = _make_params(q, kv2, dO, lse, O, idx2, dQ, dKV, sm_scale, q_start_index_s, lse_is_base2)
    lay = WorkspaceLayout()
    with torch.cuda.device(q.device):
        _raise_status(lib, lib.smla_bwd_get_workspace_layout(ctypes.byref(params), workspace.nbytes, ctypes.byref(lay)),
                      "smla_bwd_get_workspace_layout")
        stream = torch.cuda.current_stream().cuda_stream
        _raise_status(lib, lib.smla_bwd_run_stages(ctypes.byref(params), workspace.ptr, workspace.nbytes, stream, stages),
                      "smla_bwd_run_stages")
    return lay


def workspace_for(q, kv, indices, budget: int = 0) -> Workspace:
    """Allocate a workspace big enough for these shapes (at most about `budget` bytes when non-zero)."""
    lib = load_library()
    p = _Params(0, 0, 0, 0, 0, 0, 0, 0, q.shape[0], kv.shape[0], q.shape[1], indices.shape[-1], 0.0, 0, 1, None)
    need = lib.smla_bwd_workspace_size(ctypes.byref(p), budget)
    _check(need > 0, "unsupported shapes for the sparse MLA backward")
    return Workspace(need, q.device)


def device_status(workspace: Workspace) -> int:
    """Synchronise the current stream and return the library status (0 = ok, 4 = a bounded wait inside a kernel of
    any call since the last check ran out).  A recorded timeout is reported once and cleared."""
    lib = load_library()
    return lib.smla_bwd_status(workspace.ptr, torch.cuda.current_stream().cuda_stream)


def last_device_code() -> int:
    """Raw error word the last `device_status` on this thread read: 0, or 100 * kernel + site of the wait that gave up."""
    return load_library().smla_bwd_last_device_code()


def set_schedule(chunks: int, dkv_pairs: int) -> None:
    """How one pass of the backward is scheduled (`smla_bwd_set_schedule`): 0 chunks = one kernel after the other,
    -1 = chosen by the library from the head count (the default)."""
    lib = load_library()
    _raise_status(lib, lib.smla_bwd_set_schedule(int(chunks), int(dkv_pairs)), "smla_bwd_set_schedule")


def get_schedule() -> Tuple[int, int]:
    c, d = ctypes.c_int(0), ctypes.c_int(0)
    load_library().smla_bwd_get_schedule(ctypes.byref(c), ctypes.byref(d))
    return c.value, d.value


def delta(O: torch.Tensor, dO: torch.Tensor) -> torch.Tensor:
    """Delta = rowsum(O * dO), fp32 [s_q, h_q] (reference: `launch_preprocess_delta`, `mla_bwd/mla_bwd.cu:802-819`)."""
    _check(O.is_cuda and dO.is_cuda and O.dtype == torch.bfloat16 and dO.dtype == torch.bfloat16, "O, dO: CUDA bf16")
    _check(O.is_contiguous() and dO.is_contiguous() and O.shape == dO.shape and O.shape[-1] == D_V, "O, dO shape")
    lib = load_library()
    out = torch.empty(O.shape[:-1], dtype=torch.float32, device=O.device)
    with torch.cuda.device(O.device):
        st = lib.smla_bwd_delta(O.data_ptr(), dO.data_ptr(), out.data_ptr(), O.shape[0], O.shape[1],
                                torch.cuda.current_stream().cuda_stream)
    _raise_status(lib, st, "smla_bwd_delta")
    return out


class SMClock:
    """Average SM clock between two points of the current stream, from the SMs' own cycle counters."""

    def __init__(self, device):
        self.lib = load_library()
        self.n_sm = torch.cuda.get_device_properties(device).multi_processor_count
        self.a = torch.zeros(self.n_sm, 2, dtype=torch.int64, device=device)
        self.b = torch.zeros(self.n_sm, 2, dtype=torch.int64, device=device)

    def _probe(self, buf):
        buf.zero_()
        _raise_status(self.lib, self.lib.smla_clock_probe(buf.data_ptr(), self.n_sm, torch.cuda.current_stream().cuda_stream),
                      "smla_clock_probe")

    def begin(self):
        self._probe(self.a)

    def end(self):
        self._probe(self.b)

    def mhz(self) -> Optional[float]:
        """Call after a synchronise.  Mean over the SMs both probes reached of delta cycles / delta microseconds."""
        a, b = self.a.cpu(), self.b.cpu()
        ok = (a[:, 1] > 0) & (b[:, 1] > a[:, 1])
        if not ok.any():
            return None
        d = (b[ok] - a[ok]).double()
        return float((d[:, 0] / d[:, 1] * 1e3).mean().item())


def reduction_rate_gbs(s_kv: int, device, row_floats: int = 576, rows_per_cta: int = 8192, reps: int = 3) -> float:
    """GB/s at which this GPU takes fp32 reductions on random rows of a [s_kv, row_floats] buffer (one dKV), issued the
    way the dKV kernel issues them, one block per SM: the ceiling that kernel is measured against.  Best of `reps`."""
    lib = load_library()
    n_sm = torch.cuda.get_device_properties(device).multi_processor_count
    buf = torch.zeros(s_kv, row_floats, dtype=torch.float32, device=device)
    st = torch.cuda.current_stream().cuda_stream
    best = 0.0
    for i in range(reps + 1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _raise_status(lib, lib.smla_reduction_rate_probe(buf.data_ptr(), s_kv, row_floats, rows_per_cta, n_sm, st),
                      "smla_reduction_rate_probe")
        b.record()
        b.synchronize()
        if i:       # the first launch warms up
            best = max(best, n_sm * rows_per_cta * row_floats * 4 / (a.elapsed_time(b) * 1e-3) / 1e9)
    return best


def last_launch_count() -> int:
    return load_library().smla_bwd_last_launch_count()


def mla_bwd_host(q, kv, dO, lse, O, indices, device, sm_scale: Optional[float] = None,
                 q_start_index_s: Optional[int] = 0, lse_is_base2: bool = True,
                 workspace: Optional[Workspace] = None, out_dq: Optional[torch.Tensor] = None,
                 out_dkv: Optional[torch.Tensor] = None, n_chunks: int = 8) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same operator for HOST tensors (pinned memory makes the copies asynchronous).

    The query dimension is cut into `n_chunks` blocks and pipelined over three streams: block i+1 is
    copied to `device` while block i runs and the dQ of block i-1 travels back; every block adds into
    one fp32 dKV on the device, which returns last.  Returns (dQ, dKV) as host tensors (written into
    `out_dq` / `out_dkv` when given) and synchronises before returning.
    """
    dev = torch.device(device)
    s_q = q.shape[0]
    n_chunks = max(1, min(n_chunks, s_q))
    bounds = [(i * s_q) // n_chunks for i in range(n_chunks + 1)]
    if out_dq is None:
        out_dq = torch.empty(q.shape, dtype=torch.bfloat16, pin_memory=True)
    if out_dkv is None:
        out_dkv = torch.empty(kv.shape, dtype=torch.float32, pin_memory=True)
    with torch.cuda.device(dev):
        s_comp = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        s_in.wait_stream(s_comp)
        with torch.cuda.stream(s_in):
            kv_d = kv.to(dev, non_blocking=True)
        dkv_d = torch.zeros(kv.shape, dtype=torch.float32, device=dev)
        keep = []
        for c in range(n_chunks):
            r0, r1 = bounds[c], bounds[c + 1]
            if r1 == r0:
                continue
            with torch.cuda.stream(s_in):
                blk = [t[r0:r1].to(dev, non_blocking=True) for t in (q, dO, lse, O, indices)]
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            s_comp.wait_event(ev_in)
            for t in blk + [kv_d]:
                t.record_stream(s_comp)
            qs = None if q_start_index_s is None else q_start_index_s + r0
            dq_d, _ = mla_bwd(blk[0], kv_d, blk[1], blk[2], blk[3], blk[4], sm_scale=sm_scale, q_start_index_s=qs,
                              lse_is_base2=lse_is_base2, out_dkv=dkv_d, accumulate=True, workspace=workspace)
            ev_c = torch.cuda.Event()
            ev_c.record(s_comp)
            s_out.wait_event(ev_c)
            with torch.cuda.stream(s_out):
                out_dq[r0:r1].copy_(dq_d, non_blocking=True)
            dq_d.record_stream(s_out)
            keep.append((blk, dq_d))
        s_out.wait_stream(s_comp)
        with torch.cuda.stream(s_out):
            out_dkv.copy_(dkv_d, non_blocking=True)
        dkv_d.record_stream(s_out)
        s_out.synchronize()
        s_comp.synchronize()
    return out_dq, out_dkv
