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
             val_scale=None, softmax_scale=0.0, stream=None):
    """``bdattn_sdpa_fwd``.  q/out and k/v are a tensor or a list of one or two
    tensors (row segments attended as if concatenated); tensors are
    (rows, nh*hd) or (B, rows, nh*hd) torch CUDA tensors."""
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
    _check(lib().bdattn_sdpa_fwd(C.byref(p), _stream(stream)))


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
