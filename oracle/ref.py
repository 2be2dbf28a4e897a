"""ctypes front-end for ``oracle/_ref/libref.so``: brodiffusion's own
``src/dit/common.cpp`` compiled unmodified (see the Makefile beside this file).

TEST INFRASTRUCTURE ONLY.  It exists to pin the oracle restatement: tests
compare ``oracle.py`` with it, and ``tests/golden/make_ref_pin.py`` writes its
outputs into a committed fixture so that the pin also holds on hosts where the
reference tree, and therefore this library, is absent.  The product package
never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref.so")
# the brodiffusion source tree: BRODIFFUSION_REF, else the directory named reference beside this repository
REF_TREE = os.environ.get("BRODIFFUSION_REF",
                          os.path.abspath(os.path.join(_HERE, "..", "..", "reference")))
_lib = None
_fp = C.POINTER(C.c_float)


def can_build() -> bool:
    return os.path.exists(os.path.join(REF_TREE, "src", "dit", "common.cpp"))


def build(force: bool = False) -> str:
    """Compile the library from the reference tree where it lies."""
    if not can_build():
        raise RuntimeError(f"the brodiffusion source tree is not at {REF_TREE}")
    cmd = ["make", "-C", _HERE, f"REF={REF_TREE}", "_ref/libref.so"]
    if force:
        cmd.insert(3, "-B")
    subprocess.check_call(cmd, stdout=subprocess.DEVNULL)
    return LIB_PATH


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
        _lib.ref_last_error.restype = C.c_char_p
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def flux_rope_tables(txt_len, hp, wp, head_dim, axes=(16, 56, 56), theta=10000.0):
    """dit::build_axial_rope_tables (src/dit/common.cpp:116-184)."""
    L, half = txt_len + hp * wp, head_dim // 2
    cos = np.empty((L, max(half, 0)), np.float32)
    sin = np.empty_like(cos)
    ax = (C.c_int * len(axes))(*axes)
    rc = lib().ref_build_axial_rope_tables(txt_len, hp, wp, head_dim, ax, len(axes), C.c_float(theta),
                                           cos.ctypes.data_as(_fp), sin.ctypes.data_as(_fp))
    if rc != 0:
        raise RuntimeError(lib().ref_last_error().decode())
    return cos, sin


def joint_attention_traced(q, k, v, cos, sin, head_dim, num_heads, txt_len=0, bias=None, bf16=False):
    """dit::joint_attention_traced (src/dit/common.cpp:198-329): returns
    (out (L, D), head-averaged softmax map (L, L))."""
    q, qp = _f(q); k, kp = _f(k); v, vp = _f(v)
    cos, cp = _f(cos); sin, sp = _f(sin)
    L, D = q.shape
    bp = None
    if bias is not None:
        bias, bp = _f(bias)
    out = np.empty((L, D), np.float32)
    avg = np.empty((L, L), np.float32)
    rc = lib().ref_joint_attention_traced(qp, kp, vp, cp, sp, L, D, head_dim, num_heads, txt_len, bp,
                                          1 if bf16 else 0, out.ctypes.data_as(_fp), avg.ctypes.data_as(_fp))
    if rc != 0:
        raise RuntimeError(lib().ref_last_error().decode())
    return out, avg
