"""ctypes loader and numpy front-end for the CPU oracle (``oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke``
and by the CPU-baseline / reference legs of ``bench.py``.  The product package
never imports this module.

Every function takes and returns float32 numpy arrays (row-major).  The
reference lines each routine follows are cited in ``oracle.cpp``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    ):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.bdo_hardware_threads.restype = C.c_int
        _lib.bdo_flux_rope_tables.restype = C.c_int
        _lib.bdo_qwen_rope_tables.restype = C.c_int
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_ip)


def hardware_threads() -> int:
    return int(lib().bdo_hardware_threads())


# --------------------------------------------------------------------------
# bf16 / fp16 rounding helpers (round-to-nearest-even), so that the GPU and
# the oracle consume identical values.
def round_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16).reshape(x.shape)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32).reshape(b.shape)


def round_fp16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


# --------------------------------------------------------------------------
def flux_rope_tables(txt_len, hp, wp, head_dim, axes=(16, 56, 56), theta=10000.0):
    L = txt_len + hp * wp
    half = head_dim // 2
    cos = np.empty((L, half), np.float32)
    sin = np.empty((L, half), np.float32)
    ax, axp = _i(list(axes))
    r = lib().bdo_flux_rope_tables(txt_len, hp, wp, head_dim, axp, len(axes),
                                   C.c_float(theta), cos.ctypes.data_as(_fp),
                                   sin.ctypes.data_as(_fp))
    if r < 0:
        raise ValueError("build_axial_rope_tables: bad head_dim / axes_dims_rope")
    return cos, sin


def qwen_rope_tables(prefix, hp, wp, head_dim, axes=(16, 56, 56), theta=10000.0):
    """prefix: list of ("text", n) or ("image", h, w) segments."""
    kind = [0 if s[0] == "text" else 1 for s in prefix]
    n = [s[1] if s[0] == "text" else s[1] * s[2] for s in prefix]
    h = [0 if s[0] == "text" else s[1] for s in prefix]
    w = [0 if s[0] == "text" else s[2] for s in prefix]
    ka, kp = _i(kind or [0]); na, npp = _i(n or [0]); ha, hpp = _i(h or [0]); wa, wpp = _i(w or [0])
    ax, axp = _i(list(axes))
    L = lib().bdo_qwen_rope_tables(kp, npp, hpp, wpp, len(prefix), hp, wp, head_dim,
                                   axp, C.c_float(theta), None, None)
    half = head_dim // 2
    cos = np.empty((L, half), np.float32)
    sin = np.empty((L, half), np.float32)
    r = lib().bdo_qwen_rope_tables(kp, npp, hpp, wpp, len(prefix), hp, wp, head_dim,
                                   axp, C.c_float(theta), cos.ctypes.data_as(_fp),
                                   sin.ctypes.data_as(_fp))
    if r < 0:
        raise ValueError("qwen rope: axes_dims_rope must sum to head_dim")
    return cos, sin


def rms_norm_heads(x, nh, hd, gain, eps=1e-6):
    x, xp = _f(x)
    g, gp = _f(gain)
    L = x.shape[0]
    out = np.empty_like(x)
    lib().bdo_rms_norm_heads(xp, L, nh, hd, gp, C.c_float(eps), out.ctypes.data_as(_fp))
    return out


def rope_apply(x, nh, hd, cos, sin, pair_mode=0):
    x, xp = _f(x)
    c, cp = _f(cos)
    s, sp = _f(sin)
    out = np.empty_like(x)
    lib().bdo_rope_apply(xp, x.shape[0], nh, hd, cp, sp, pair_mode,
                         out.ctypes.data_as(_fp))
    return out


def sdpa(q, k, v, nh, *, mask_mode=0, seg_id=None, seg_is_image=None, key_mask=None,
         bias=None, bias_row0=0, rows=None, precise=True, nthreads=0,
         want_avg=False):
    q, qp = _f(q); k, kp = _f(k); v, vp = _f(v)
    Lq, D = q.shape
    Lk = k.shape[0]
    hd = D // nh
    sidp = sisp = kmp = bp = rp = None
    bias_cols = 0
    if seg_id is not None:
        seg_id, sidp = _i(seg_id)
        seg_is_image, sisp = _i(seg_is_image)
    if key_mask is not None:
        key_mask, kmp = _f(key_mask)
    if bias is not None:
        bias, bp = _f(bias)
        bias_cols = bias.shape[1]
    n_rows = Lq
    if rows is not None:
        rows, rp = _i(rows)
        n_rows = rows.shape[0]
    out = np.empty((n_rows, D), np.float32)
    avg = np.empty((n_rows, Lk), np.float32) if want_avg else None
    lib().bdo_sdpa(qp, Lq, kp, vp, Lk, nh, hd, mask_mode, sidp, sisp, kmp, bp,
                   bias_row0, bias_cols, rp, n_rows, 1 if precise else 0, nthreads,
                   out.ctypes.data_as(_fp),
                   avg.ctypes.data_as(_fp) if want_avg else None)
    return (out, avg) if want_avg else out


def linear(x, w, b=None, nthreads=0):
    x, xp = _f(x); w, wp = _f(w)
    bp = None
    if b is not None:
        b, bp = _f(np.reshape(b, -1))
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), np.float32)
    lib().bdo_linear(xp, wp, bp, M, N, K, nthreads, y.ctypes.data_as(_fp))
    return y


def sana_linear_attn(q, k, v, nh, hd, eps=1e-15, sz_in=None, w_in=0.0,
                     want_sz=False, nthreads=0):
    """q, k, v: channel-major (D, N)."""
    q, qp = _f(q); k, kp = _f(k); v, vp = _f(v)
    D, N = q.shape
    szp = None
    if sz_in is not None:
        sz_in, szp = _f(sz_in)
    szo = np.empty((nh, hd + 1, hd), np.float32) if want_sz else None
    out = np.empty((D, N), np.float32)
    lib().bdo_sana_linear_attn(qp, kp, vp, nh, hd, N, C.c_float(eps), szp,
                               C.c_float(w_in),
                               szo.ctypes.data_as(_fp) if want_sz else None,
                               nthreads, out.ctypes.data_as(_fp))
    return (out, szo) if want_sz else out


def linear_geglu(x, w, b=None, nthreads=0):
    x, xp = _f(x); w, wp = _f(w)
    bp = None
    if b is not None:
        b, bp = _f(np.reshape(b, -1))
    B, D_in = x.shape
    D_out = w.shape[0] // 2
    y = np.empty((B, D_out), np.float32)
    lib().bdo_linear_geglu(xp, wp, bp, B, D_in, D_out, nthreads, y.ctypes.data_as(_fp))
    return y


# --------------------------------------------------------------------------
# Compositions that mirror the reference call sites.

def joint_attention(Q, K, V, cos, sin, head_dim, num_heads, pair_mode=0, **kw):
    """dit::joint_attention (src/dit/common.cpp:188-196): rope(Q), rope(K), sdpa."""
    Qr = rope_apply(Q, num_heads, head_dim, cos, sin, pair_mode)
    Kr = rope_apply(K, num_heads, head_dim, cos, sin, pair_mode)
    return sdpa(Qr, Kr, V, num_heads, **kw)


def gqa_attention_masked(Q, K, V, cos, sin, head_dim, num_q_heads, num_kv_heads, key_mask=None, **kw):
    """dit::gqa_attention_masked (src/dit/common.cpp:331-377): optional rope of Q
    (num_q_heads) and K (num_kv_heads), then the K/V heads are widened so that
    query head h reads K/V head h // group (common.cpp:361-375) and plain
    attention runs on the widened tensors."""
    if num_q_heads <= 0 or num_kv_heads <= 0 or num_q_heads % num_kv_heads:
        raise ValueError("gqa_attention_masked: num_kv_heads must divide num_q_heads")
    Qr, Kr = np.asarray(Q, np.float32), np.asarray(K, np.float32)
    if cos is not None and sin is not None:
        Qr = rope_apply(Qr, num_q_heads, head_dim, cos, sin)
        Kr = rope_apply(Kr, num_kv_heads, head_dim, cos, sin)
    group = num_q_heads // num_kv_heads
    L = Kr.shape[0]
    widen = lambda x: np.repeat(np.asarray(x, np.float32).reshape(L, num_kv_heads, head_dim), group, axis=1) \
        .reshape(L, num_q_heads * head_dim)
    return sdpa(Qr, widen(Kr), widen(V), num_q_heads, key_mask=key_mask, **kw)


def prefix_cache_scale(t, scale, round_fn):
    """QwenImage21PrefixCache::scale_kv on one cached tensor
    (src/dit/qwenimage21_hooks.cpp:79-99): t *= scale, stored at the cache dtype
    (round_fn rounds FP32 to that dtype)."""
    return round_fn(np.float32(scale) * np.asarray(t, np.float32))


def prefix_cache_blend(t, other, alpha, round_fn):
    """QwenImage21PrefixCache::blend_from on one cached tensor
    (src/dit/qwenimage21_hooks.cpp:101-124): t = (1 - alpha) * t + alpha * other."""
    keep = np.float32(1.0) - np.float32(alpha)
    return round_fn(keep * np.asarray(t, np.float32) + np.float32(alpha) * np.asarray(other, np.float32))


def block_causal_tables(segments):
    """segments: list of ("text"|"image", n_tokens) incl. the target image last.
    Returns (seg_id per token, is_image per segment)."""
    seg_id, is_img = [], []
    for i, s in enumerate(segments):
        seg_id += [i] * s[1]
        is_img.append(0 if s[0] == "text" else 1)
    return np.asarray(seg_id, np.int32), np.asarray(is_img, np.int32)


def qkvo_attention(X, Ctx, Wq, Wk, Wv, Wo, bo, num_heads, bq=None, bk=None, bv=None,
                   key_mask=None, causal=False):
    """brotensor flash_attention_qkvo_forward as called from
    src/unet_blocks.cpp:264-271,320-327: project, attend, project out."""
    src = X if Ctx is None else Ctx
    q = linear(X, Wq, bq)
    k = linear(src, Wk, bk)
    v = linear(src, Wv, bv)
    o = sdpa(q, k, v, num_heads, mask_mode=1 if causal else 0, key_mask=key_mask)
    return linear(o, Wo, bo)
