"""brodiffusion_b200 — B200 (sm_100a) denoiser-attention kernels behind a C ABI.

The product is ``libbdattn.so`` (built from ``csrc/`` by ``_build.py``); its
entry points are declared in ``include/bdattn.h``.  This module is the thin
ctypes binding used by the tests and the bench: it passes raw device pointers
of ``torch`` tensors (torch is only the allocator / stream provider here) and
raises :class:`BdattnError` with the library's message when a call fails.

There is no CPU path and no fallback: loading fails loudly when the shared
library is missing, and every operator fails when no sm_100 device is current.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

__all__ = [
    "BdattnError", "lib", "lib_path", "F32", "F16", "BF16", "MASK_NONE", "MASK_CAUSAL",
    "ROPE_INTERLEAVED", "ROPE_HALF_SPLIT", "SdpaParams", "NormRopeJob", "sdpa_fwd",
    "rmsnorm_rope", "linear_attn_relu_fwd", "rope_tables_flux", "rope_tables_qwen", "RopeSegment", "device_status", "last_error",
]

F32, F16, BF16 = 0, 1, 2
MASK_NONE, MASK_CAUSAL = 0, 1
STATUS_WAIT_TIMEOUT, STATUS_BAD_ARGS = 1, 2
ROPE_INTERLEAVED, ROPE_HALF_SPLIT = 0, 1


class BdattnError(RuntimeError):
    """A bdattn entry point returned -1; the text is bdattn_last_error()."""


class SdpaParams(C.Structure):
    """Mirror of ``bdattn_sdpa_params`` (include/bdattn.h)."""
    _fields_ = [
        ("dtype", C.c_int), ("batch", C.c_int), ("num_heads", C.c_int), ("head_dim", C.c_int),
        ("n_q_seg", C.c_int),
        ("q", C.c_void_p * 2), ("o", C.c_void_p * 2), ("q_rows", C.c_int * 2),
        ("q_ld", C.c_longlong * 2), ("o_ld", C.c_longlong * 2),
        ("q_batch_stride", C.c_longlong * 2), ("o_batch_stride", C.c_longlong * 2),
        ("n_kv_seg", C.c_int),
        ("k", C.c_void_p * 2), ("v", C.c_void_p * 2), ("kv_rows", C.c_int * 2),
        ("k_ld", C.c_longlong * 2), ("v_ld", C.c_longlong * 2),
        ("k_batch_stride", C.c_longlong * 2), ("v_batch_stride", C.c_longlong * 2),
        ("mask_mode", C.c_int),
        ("key_mask", C.c_void_p), ("key_scale", C.c_void_p), ("val_scale", C.c_void_p),
        ("softmax_scale", C.c_float),
        ("num_kv_heads", C.c_int),
        ("q_gain", C.c_void_p * 2), ("q_gain_dtype", C.c_int), ("q_eps", C.c_float),
        ("q_cos", C.c_void_p), ("q_sin", C.c_void_p), ("q_rope_row0", C.c_int),
    ]


class NormRopeJob(C.Structure):
    """Mirror of ``bdattn_norm_rope_job`` (include/bdattn.h)."""
    _fields_ = [
        ("x", C.c_void_p), ("out", C.c_void_p), ("rows", C.c_int),
        ("x_ld", C.c_longlong), ("out_ld", C.c_longlong),
        ("gain", C.c_void_p), ("gain_dtype", C.c_int),
        ("cos", C.c_void_p), ("sin", C.c_void_p), ("rope_row0", C.c_int),
    ]


class RopeSegment(C.Structure):
    """Mirror of ``bdattn_rope_segment`` (include/bdattn.h)."""
    _fields_ = [("kind", C.c_int), ("n_tokens", C.c_int), ("h", C.c_int), ("w", C.c_int)]


class TraceParams(C.Structure):
    """Mirror of ``bdattn_trace_params`` (include/bdattn.h)."""
    _fields_ = [
        ("bias", C.c_void_p), ("bias_row0", C.c_int), ("bias_rows", C.c_int), ("bias_cols", C.c_int),
        ("bias_ld", C.c_longlong),
        ("attn_avg", C.c_void_p), ("map_row0", C.c_int), ("map_rows", C.c_int), ("map_cols", C.c_int),
        ("map_ld", C.c_longlong),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class QkvProjParams(C.Structure):
    """Mirror of ``bdattn_qkv_proj_params`` (include/bdattn.h)."""
    _fields_ = [
        ("dtype", C.c_int), ("num_heads", C.c_int), ("head_dim", C.c_int),
        ("x", C.c_void_p), ("rows", C.c_int), ("in_features", C.c_int), ("x_ld", C.c_longlong),
        ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
        ("bq", C.c_void_p), ("bk", C.c_void_p), ("bv", C.c_void_p),
        ("gain_q", C.c_void_p), ("gain_k", C.c_void_p), ("gain_dtype", C.c_int), ("eps", C.c_float),
        ("cos", C.c_void_p), ("sin", C.c_void_p), ("rope_row0", C.c_int),
        ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("v_out", C.c_void_p),
        ("q_ld", C.c_longlong), ("k_ld", C.c_longlong), ("v_ld", C.c_longlong),
    ]


class QkvoParams(C.Structure):
    """Mirror of ``bdattn_qkvo_params`` (include/bdattn.h)."""
    _fields_ = [
        ("dtype", C.c_int), ("num_heads", C.c_int), ("inner_dim", C.c_int), ("causal", C.c_int),
        ("x", C.c_void_p), ("x_rows", C.c_int), ("x_cols", C.c_int), ("x_ld", C.c_longlong),
        ("ctx", C.c_void_p), ("ctx_rows", C.c_int), ("ctx_cols", C.c_int), ("ctx_ld", C.c_longlong),
        ("wq", C.c_void_p), ("bq", C.c_void_p), ("wk", C.c_void_p), ("bk", C.c_void_p),
        ("wv", C.c_void_p), ("bv", C.c_void_p), ("wo", C.c_void_p), ("bo", C.c_void_p),
        ("k_cached", C.c_void_p), ("v_cached", C.c_void_p), ("kv_rows", C.c_int),
        ("k_ld", C.c_longlong), ("v_ld", C.c_longlong),
        ("key_mask", C.c_void_p),
        ("out", C.c_void_p), ("out_cols", C.c_int), ("out_ld", C.c_longlong),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def lib():
    """Load ``libbdattn.so`` (no build is attempted here)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise BdattnError(
                f"{path} is missing: build it with `python -m brodiffusion_b200._build` "
                "(there is no fallback implementation)")
        L = C.CDLL(path)
        L.bdattn_version.restype = C.c_int
        L.bdattn_last_error.restype = C.c_char_p
        L.bdattn_device_status.argtypes = [C.POINTER(C.c_int), C.c_int]
        L.bdattn_sdpa_fwd.argtypes = [C.POINTER(SdpaParams), C.c_void_p]
        L.bdattn_sdpa_fwd_allgather.argtypes = [C.POINTER(SdpaParams), C.POINTER(C.c_void_p),
                                                C.POINTER(C.c_void_p), C.c_int, C.c_void_p]
        L.bdattn_sdpa_fwd_allgather_multicast.argtypes = [C.POINTER(SdpaParams), C.c_void_p, C.c_void_p,
                                                          C.c_void_p]
        L.bdattn_mgpu_init.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int]
        L.bdattn_mgpu_destroy.argtypes = [C.c_void_p]
        L.bdattn_mgpu_size.argtypes = [C.c_void_p]
        L.bdattn_mgpu_barrier.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.bdattn_mgpu_sdpa_fwd_headsharded.argtypes = [C.c_void_p, C.c_int, C.POINTER(SdpaParams),
                                                       C.POINTER(C.c_void_p), C.c_longlong, C.c_longlong,
                                                       C.c_int, C.c_void_p]
        L.bdattn_sdpa_traced_workspace_bytes.restype = C.c_size_t
        L.bdattn_sdpa_traced_workspace_bytes.argtypes = [C.c_int, C.c_int]
        L.bdattn_sdpa_traced_fwd.argtypes = [C.POINTER(SdpaParams), C.POINTER(TraceParams), C.c_void_p]
        L.bdattn_rmsnorm_rope.argtypes = [C.POINTER(NormRopeJob), C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_float, C.c_int, C.c_void_p]
        L.bdattn_linear_attn_relu_fwd.argtypes = [
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
            C.c_int, C.c_longlong, C.c_longlong, C.c_float, C.c_void_p, C.c_float, C.c_void_p,
            C.c_void_p]
        L.bdattn_rope_tables_flux.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int,
                                              C.POINTER(C.c_int), C.c_int, C.c_float,
                                              C.c_void_p, C.c_void_p, C.c_void_p]
        L.bdattn_rope_rows_qwen.argtypes = [C.POINTER(RopeSegment), C.c_int, C.c_int, C.c_int]
        L.bdattn_rope_tables_qwen.argtypes = [C.POINTER(RopeSegment), C.c_int, C.c_int, C.c_int,
                                              C.c_int, C.POINTER(C.c_int), C.c_float,
                                              C.c_void_p, C.c_void_p, C.c_void_p]
        L.bdattn_qkvo_workspace_bytes.restype = C.c_size_t
        L.bdattn_qkvo_workspace_bytes.argtypes = [C.c_int] * 4
        L.bdattn_qkvo_fwd.argtypes = [C.POINTER(QkvoParams), C.c_void_p]
        L.bdattn_qkvo_static_capacity.restype = C.c_size_t
        L.bdattn_qkvo_fwd_static.argtypes = [C.POINTER(QkvoParams), C.c_void_p]
        L.bdattn_qkv_norm_rope_fwd.argtypes = [C.POINTER(QkvProjParams), C.c_void_p]
        L.bdattn_project_kv.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_longlong, C.c_int, C.c_int, C.c_void_p]
        L.bdattn_linear_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                        C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong,
                                        C.c_longlong, C.c_void_p]
        L.bdattn_linear_geglu_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.bdattn_add_inplace.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]
        L.bdattn_axpby_inplace.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_float, C.c_float,
                                           C.c_int, C.c_void_p]
        L.bdattn_add_row_bias.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong,
                                          C.c_int, C.c_void_p]
        _lib = L
    return _lib


def last_error() -> str:
    return lib().bdattn_last_error().decode()


def _check(rc: int) -> None:
    if rc != 0:
        raise BdattnError(last_error())


def _stream(stream=None):
    """Raw cudaStream_t of a torch stream (default: torch's current stream)."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


def _dtype_code(t) -> int:
    import torch
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.float32:
        return F32
    raise BdattnError(f"unsupported tensor dtype {t.dtype}")


def _rows2d(t):
    """(ptr, rows, ld, batch_stride, batch) of a (rows, cols) or (B, rows, cols) tensor."""
    if t.dim() == 2:
        if t.stride(1) != 1:
            raise BdattnError("tensor columns must be contiguous")
        return t.data_ptr(), t.shape[0], t.stride(0), t.shape[0] * t.stride(0), 1
    if t.dim() == 3:
        if t.stride(2) != 1:
            raise BdattnError("tensor columns must be contiguous")
        return t.data_ptr(), t.shape[1], t.stride(1), t.stride(0), t.shape[0]
    raise BdattnError("expected a 2-D or 3-D tensor")


def device_status(clear: bool = True) -> int:
    v = C.c_int(0)
    _check(lib().bdattn_device_status(C.byref(v), 1 if clear else 0))
    return v.value


def sdpa_fwd(q, k, v, out, num_heads, *, mask_mode=MASK_NONE, key_mask=None, key_scale=None,
             val_scale=None, softmax_scale=0.0, num_kv_heads=0, q_norm=None, stream=None,
             peer_out_ptrs=None, multicast_out_ptrs=None, _trace=None, _mgpu=None):
    """``bdattn_sdpa_fwd``.  q/out and k/v are a tensor or a list of one or two
    tensors (row segments attended as if concatenated); tensors are
    (rows, nh*hd) or (B, rows, nh*hd) torch CUDA tensors.
    ``peer_out_ptrs`` (list per output segment of lists of raw device pointers
    on other GPUs) selects ``bdattn_sdpa_fwd_allgather``; ``multicast_out_ptrs``
    (one NVLink multicast address per output segment) selects
    ``bdattn_sdpa_fwd_allgather_multicast``."""
    qs = list(q) if isinstance(q, (list, tuple)) else [q]
    os_ = list(out) if isinstance(out, (list, tuple)) else [out]
    ks = list(k) if isinstance(k, (list, tuple)) else [k]
    vs = list(v) if isinstance(v, (list, tuple)) else [v]
    if len(qs) != len(os_) or len(ks) != len(vs):
        raise BdattnError("q/out and k/v segment lists must have equal lengths")
    p = SdpaParams()
    p.dtype = _dtype_code(qs[0])
    p.num_heads = num_heads
    p.head_dim = qs[0].shape[-1] // num_heads
    p.n_q_seg = len(qs)
    p.n_kv_seg = len(ks)
    for i, (qq, oo) in enumerate(zip(qs, os_)):
        ptr, rows, ld, bs, B = _rows2d(qq)
        optr, orows, old, obs, oB = _rows2d(oo)
        if orows != rows or oB != B:
            raise BdattnError("out segment shape differs from q segment shape")
        p.q[i], p.o[i], p.q_rows[i] = ptr, optr, rows
        p.q_ld[i], p.o_ld[i] = ld, old
        p.q_batch_stride[i], p.o_batch_stride[i] = bs, obs
        p.batch = B
    for i, (kk, vv) in enumerate(zip(ks, vs)):
        ptr, rows, ld, bs, B = _rows2d(kk)
        vptr, vrows, vld, vbs, vB = _rows2d(vv)
        if vrows != rows:
            raise BdattnError("k and v segment row counts differ")
        p.k[i], p.v[i], p.kv_rows[i] = ptr, vptr, rows
        p.k_ld[i], p.v_ld[i] = ld, vld
        p.k_batch_stride[i], p.v_batch_stride[i] = bs, vbs
    p.mask_mode = mask_mode
    p.key_mask = key_mask.data_ptr() if key_mask is not None else None
    p.key_scale = key_scale.data_ptr() if key_scale is not None else None
    p.val_scale = val_scale.data_ptr() if val_scale is not None else None
    p.softmax_scale = softmax_scale
    p.num_kv_heads = num_kv_heads
    if q_norm is not None:
        # dict(gain=tensor | [per-segment tensors] | None, cos=, sin=, rope_row0=0, eps=1e-6):
        # RMSNorm + RoPE of the query rows inside the attention kernel
        gains = q_norm.get("gain")
        gains = list(gains) if isinstance(gains, (list, tuple)) else [gains] * len(qs)
        for i, gt in enumerate(gains[:2]):
            p.q_gain[i] = _ptr(gt)
        g0 = next((gt for gt in gains if gt is not None), None)
        p.q_gain_dtype = _dtype_code(g0) if g0 is not None else F32
        p.q_eps = q_norm.get("eps", 1e-6)
        p.q_cos, p.q_sin = _ptr(q_norm.get("cos")), _ptr(q_norm.get("sin"))
        p.q_rope_row0 = q_norm.get("rope_row0", 0)
    if _trace is not None:
        _check(lib().bdattn_sdpa_traced_fwd(C.byref(p), C.byref(_trace), _stream(stream)))
        return
    if _mgpu is not None:
        ctx, rank, replica_ptrs, replica_ld, replica_bs, total_heads = _mgpu
        arr = (C.c_void_p * len(replica_ptrs))(*replica_ptrs)
        _check(lib().bdattn_mgpu_sdpa_fwd_headsharded(ctx, rank, C.byref(p), arr, replica_ld, replica_bs,
                                                      total_heads, _stream(stream)))
        return
    if multicast_out_ptrs:
        m1 = multicast_out_ptrs[1] if len(multicast_out_ptrs) > 1 else None
        _check(lib().bdattn_sdpa_fwd_allgather_multicast(C.byref(p), multicast_out_ptrs[0], m1, _stream(stream)))
        return
    if peer_out_ptrs:
        n = len(peer_out_ptrs[0])
        a0 = (C.c_void_p * max(n, 1))(*peer_out_ptrs[0])
        a1 = (C.c_void_p * max(n, 1))(*(peer_out_ptrs[1] if len(peer_out_ptrs) > 1 else [None] * n))
        _check(lib().bdattn_sdpa_fwd_allgather(C.byref(p), a0, a1, n, _stream(stream)))
        return
    _check(lib().bdattn_sdpa_fwd(C.byref(p), _stream(stream)))


class MultiGpu:
    """``bdattn_mgpu_*``: several GPUs driven from one process, one host thread per
    GPU.  ``replicas`` are the callers' full-output tensors, one per GPU."""

    def __init__(self, devices):
        self.devices = list(devices)
        h = C.c_void_p()
        arr = (C.c_int * len(self.devices))(*self.devices)
        _check(lib().bdattn_mgpu_init(C.byref(h), arr, len(self.devices)))
        self.handle = h

    def size(self) -> int:
        return int(lib().bdattn_mgpu_size(self.handle))

    def sdpa_fwd_headsharded(self, rank, q, k, v, replicas, total_heads, **kw):
        """q, k, v: this rank's head columns (tensor or segment lists as for
        ``sdpa_fwd``); replicas: list of (B, L, D) or (L, D) tensors, one per GPU."""
        r0 = replicas[0]
        ld = r0.stride(-2)
        bs = r0.stride(0) if r0.dim() == 3 else 0
        qs = list(q) if isinstance(q, (list, tuple)) else [q]
        dummy = [t for t in qs]          # shapes only: the library derives the output pointers
        sdpa_fwd(q, k, v, dummy if isinstance(q, (list, tuple)) else dummy[0], total_heads // len(replicas),
                 _mgpu=(self.handle, rank, [t.data_ptr() for t in replicas], ld, bs, total_heads), **kw)

    def barrier(self, rank, timeout_ms=0, stream=None):
        _check(lib().bdattn_mgpu_barrier(self.handle, rank, timeout_ms, _stream(stream)))

    def destroy(self):
        if self.handle is not None:
            lib().bdattn_mgpu_destroy(self.handle)
            self.handle = None


def rmsnorm_rope(jobs, num_heads, head_dim, *, eps=1e-6, pair_mode=ROPE_INTERLEAVED, stream=None):
    """``bdattn_rmsnorm_rope``.  jobs: list of dicts with keys x, out and
    optional gain, cos, sin, rope_row0 (torch CUDA tensors)."""
    arr = (NormRopeJob * len(jobs))()
    dtype = _dtype_code(jobs[0]["x"])
    for i, j in enumerate(jobs):
        x, out = j["x"], j["out"]
        arr[i].x, arr[i].out = x.data_ptr(), out.data_ptr()
        arr[i].rows = x.shape[0]
        arr[i].x_ld, arr[i].out_ld = x.stride(0), out.stride(0)
        g = j.get("gain")
        arr[i].gain = g.data_ptr() if g is not None else None
        arr[i].gain_dtype = _dtype_code(g) if g is not None else F32
        c, s = j.get("cos"), j.get("sin")
        arr[i].cos = c.data_ptr() if c is not None else None
        arr[i].sin = s.data_ptr() if s is not None else None
        arr[i].rope_row0 = j.get("rope_row0", 0)
    _check(lib().bdattn_rmsnorm_rope(arr, len(jobs), dtype, num_heads, head_dim, eps, pair_mode,
                                     _stream(stream)))


def rope_tables_flux(txt_len, hp, wp, head_dim, axes=(16, 56, 56), theta=10000.0, *,
                     device=None, stream=None):
    """``bdattn_rope_tables_flux`` -> (cos, sin) FP32 CUDA tensors (L, head_dim/2)."""
    import torch
    L = txt_len + hp * wp
    device = device or torch.device("cuda", torch.cuda.current_device())
    cos = torch.empty(max(L, 1), head_dim // 2, device=device, dtype=torch.float32)
    sin = torch.empty_like(cos)
    ax = (C.c_int * len(axes))(*axes)
    _check(lib().bdattn_rope_tables_flux(txt_len, hp, wp, head_dim, ax, len(axes), theta,
                                         cos.data_ptr(), sin.data_ptr(), _stream(stream)))
    return cos, sin


def rope_tables_qwen(prefix, hp, wp, head_dim, axes=(16, 56, 56), theta=10000.0, *,
                     device=None, stream=None):
    """``bdattn_rope_tables_qwen``.  prefix: list of ("text", n) / ("image", h, w)."""
    import torch
    segs = (RopeSegment * max(len(prefix), 1))()
    for i, s in enumerate(prefix):
        if s[0] == "text":
            segs[i].kind, segs[i].n_tokens = 0, s[1]
        else:
            segs[i].kind, segs[i].h, segs[i].w = 1, s[1], s[2]
    rows = lib().bdattn_rope_rows_qwen(segs, len(prefix), hp, wp)
    device = device or torch.device("cuda", torch.cuda.current_device())
    cos = torch.empty(max(rows, 1), head_dim // 2, device=device, dtype=torch.float32)
    sin = torch.empty_like(cos)
    ax = (C.c_int * 3)(*axes)
    _check(lib().bdattn_rope_tables_qwen(segs, len(prefix), hp, wp, head_dim, ax, theta,
                                         cos.data_ptr(), sin.data_ptr(), _stream(stream)))
    return cos, sin


def linear_attn_relu_fwd(q, k, v, out, num_heads, head_dim, *, eps=1e-15, sz_in=None, w_in=0.0,
                         sz_out=None, stream=None):
    """``bdattn_linear_attn_relu_fwd``.  q/k/v/out: channel-major (D, N) or
    (B, D, N) torch CUDA tensors."""
    ptr, rows, ld, bs, B = _rows2d(q)
    n_tokens = q.shape[-1]
    for t in (k, v, out):
        p2, r2, ld2, bs2, B2 = _rows2d(t)
        if (r2, ld2, bs2, B2) != (rows, ld, bs, B):
            raise BdattnError("q, k, v and out must share shape and strides")
    _check(lib().bdattn_linear_attn_relu_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _dtype_code(q), B, num_heads,
        head_dim, n_tokens, ld, bs, eps, sz_in.data_ptr() if sz_in is not None else None, w_in,
        sz_out.data_ptr() if sz_out is not None else None, _stream(stream)))


def _ptr(t):
    return t.data_ptr() if t is not None else None


def qkvo_workspace_bytes(q_rows, kv_rows, num_heads, head_dim) -> int:
    return int(lib().bdattn_qkvo_workspace_bytes(q_rows, kv_rows, num_heads, head_dim))


def qkvo_fwd(x, ctx, wq, wk, wv, wo, bo, num_heads, out, workspace, *, bq=None, bk=None, bv=None,
             k_cached=None, v_cached=None, key_mask=None, causal=False, stream=None):
    """``bdattn_qkvo_fwd``: the reference's flash_attention_qkvo_forward, or
    flash_attention_q_with_kv_cached_forward when k_cached / v_cached are given.
    ``workspace=None`` calls ``bdattn_qkvo_fwd_static`` instead, which keeps its
    scratch in a fixed array inside the library (for callers that may not
    allocate device memory; see include/bdattn.h for its limits)."""
    p = QkvoParams()
    p.dtype = _dtype_code(x)
    p.num_heads = num_heads
    p.inner_dim = wq.shape[0]
    p.causal = 1 if causal else 0
    p.x, p.x_rows, p.x_cols, p.x_ld = x.data_ptr(), x.shape[0], x.shape[1], x.stride(0)
    if ctx is not None:
        p.ctx, p.ctx_rows, p.ctx_cols, p.ctx_ld = ctx.data_ptr(), ctx.shape[0], ctx.shape[1], ctx.stride(0)
    p.wq, p.bq, p.wk, p.bk = _ptr(wq), _ptr(bq), _ptr(wk), _ptr(bk)
    p.wv, p.bv, p.wo, p.bo = _ptr(wv), _ptr(bv), _ptr(wo), _ptr(bo)
    if k_cached is not None:
        p.k_cached, p.v_cached = k_cached.data_ptr(), v_cached.data_ptr()
        p.kv_rows, p.k_ld, p.v_ld = k_cached.shape[0], k_cached.stride(0), v_cached.stride(0)
    p.key_mask = _ptr(key_mask)
    p.out, p.out_cols, p.out_ld = out.data_ptr(), out.shape[1], out.stride(0)
    if workspace is None:
        _check(lib().bdattn_qkvo_fwd_static(C.byref(p), _stream(stream)))
        return
    p.workspace = workspace.data_ptr()
    p.workspace_bytes = workspace.numel() * workspace.element_size()
    _check(lib().bdattn_qkvo_fwd(C.byref(p), _stream(stream)))


def qkvo_static_capacity() -> int:
    return int(lib().bdattn_qkvo_static_capacity())


def project_kv(ctx, wk, wv, k_out, v_out, *, bk=None, bv=None, stream=None):
    """``bdattn_project_kv`` (flash_attention_project_kv)."""
    _check(lib().bdattn_project_kv(ctx.data_ptr(), ctx.shape[0], ctx.shape[1], ctx.stride(0),
                                   wk.data_ptr(), _ptr(bk), wv.data_ptr(), _ptr(bv),
                                   k_out.data_ptr(), v_out.data_ptr(), k_out.stride(0), wk.shape[0],
                                   _dtype_code(ctx), _stream(stream)))


def linear_fwd(x, w, bias, y, *, stream=None):
    """``bdattn_linear_fwd``: y = x @ w.T + bias."""
    _check(lib().bdattn_linear_fwd(x.data_ptr(), w.data_ptr(), _ptr(bias), y.data_ptr(),
                                   _dtype_code(x), x.shape[0], w.shape[0], x.shape[1], x.stride(0),
                                   w.stride(0), y.stride(0), _stream(stream)))


def linear_geglu_fwd(x, w, bias, y, *, stream=None):
    """``bdattn_linear_geglu_fwd`` (fused_linear_geglu)."""
    _check(lib().bdattn_linear_geglu_fwd(x.data_ptr(), w.data_ptr(), _ptr(bias), y.data_ptr(),
                                         _dtype_code(x), x.shape[0], x.shape[1], w.shape[0] // 2,
                                         _stream(stream)))


def add_inplace(y, x, *, stream=None):
    """``bdattn_add_inplace`` (add_inplace_vec): y += x, both dense."""
    if y.shape != x.shape or not y.is_contiguous() or not x.is_contiguous():
        raise BdattnError("add_inplace_vec: Y and X must be dense and of equal shape")
    _check(lib().bdattn_add_inplace(y.data_ptr(), x.data_ptr(), y.numel(), _dtype_code(y),
                                    _stream(stream)))


def axpby_inplace(y, x, a, b=0.0, *, stream=None):
    """``bdattn_axpby_inplace``: y = a*y + b*x in place (x may be None: y = a*y).
    The prefix-cache ``scale_kv`` / ``blend_from`` operations."""
    if not y.is_contiguous() or (x is not None and (x.shape != y.shape or not x.is_contiguous())):
        raise BdattnError("axpby_inplace: Y and X must be dense and of equal shape")
    _check(lib().bdattn_axpby_inplace(y.data_ptr(), _ptr(x), y.numel(), a, b, _dtype_code(y), _stream(stream)))


def add_row_bias(y, bias, *, stream=None):
    """``bdattn_add_row_bias`` (add_inplace_row_bias): y[i, j] += bias[j]."""
    if bias.numel() != y.shape[1]:
        raise BdattnError("add_inplace_row_bias: bias length must equal the column count")
    _check(lib().bdattn_add_row_bias(y.data_ptr(), bias.data_ptr(), y.shape[0], y.shape[1],
                                     y.stride(0), _dtype_code(y), _stream(stream)))


def sdpa_traced_fwd(q, k, v, out, num_heads, *, bias=None, bias_row0=0, map_row0=0, map_rows=0,
                    map_cols=0, mask_mode=MASK_NONE, key_mask=None, stream=None):
    """``bdattn_sdpa_traced_fwd``: attention with an optional FP32 logit bias on
    queries [bias_row0, bias_row0 + bias.shape[0]) x keys [0, bias.shape[1]) and,
    when map_rows > 0, the head-averaged softmax block (map_rows, map_cols)
    returned as an FP32 tensor."""
    import torch
    qs = list(q) if isinstance(q, (list, tuple)) else [q]
    Lq = sum(t.shape[-2] for t in qs)
    t = TraceParams()
    if bias is not None:
        t.bias, t.bias_row0 = bias.data_ptr(), bias_row0
        t.bias_rows, t.bias_cols, t.bias_ld = bias.shape[0], bias.shape[1], bias.stride(0)
    amap = None
    if map_rows > 0:
        amap = torch.empty(map_rows, map_cols, device=qs[0].device, dtype=torch.float32)
        t.attn_avg, t.map_row0, t.map_rows, t.map_cols, t.map_ld = amap.data_ptr(), map_row0, map_rows, map_cols, map_cols
    ws = torch.empty(int(lib().bdattn_sdpa_traced_workspace_bytes(num_heads, Lq)), device=qs[0].device,
                     dtype=torch.uint8)
    t.workspace, t.workspace_bytes = ws.data_ptr(), ws.numel()
    sdpa_fwd(q, k, v, out, num_heads, mask_mode=mask_mode, key_mask=key_mask, stream=stream, _trace=t)
    return amap


def qkv_norm_rope_fwd(x, wq, wk, wv, q_out, k_out, v_out, num_heads, head_dim, *, gain_q=None,
                      gain_k=None, cos=None, sin=None, rope_row0=0, eps=1e-6, bq=None, bk=None,
                      bv=None, stream=None):
    """``bdattn_qkv_norm_rope_fwd``: Q/K/V projections with per-head RMSNorm and
    RoPE in the GEMM epilogue."""
    p = QkvProjParams()
    p.dtype, p.num_heads, p.head_dim = _dtype_code(x), num_heads, head_dim
    p.x, p.rows, p.in_features, p.x_ld = x.data_ptr(), x.shape[0], x.shape[1], x.stride(0)
    p.wq, p.wk, p.wv = _ptr(wq), _ptr(wk), _ptr(wv)
    p.bq, p.bk, p.bv = _ptr(bq), _ptr(bk), _ptr(bv)
    p.gain_q, p.gain_k = _ptr(gain_q), _ptr(gain_k)
    g = gain_q if gain_q is not None else gain_k
    p.gain_dtype = _dtype_code(g) if g is not None else F32
    p.eps = eps
    p.cos, p.sin, p.rope_row0 = _ptr(cos), _ptr(sin), rope_row0
    p.q_out, p.k_out, p.v_out = _ptr(q_out), _ptr(k_out), _ptr(v_out)
    p.q_ld = q_out.stride(0) if q_out is not None else 0
    p.k_ld = k_out.stride(0) if k_out is not None else 0
    p.v_ld = v_out.stride(0) if v_out is not None else 0
    _check(lib().bdattn_qkv_norm_rope_fwd(C.byref(p), _stream(stream)))
