"""Pins the CPU oracle to the reference's own arithmetic.

brodiffusion's ``src/dit/common.cpp`` holds, in plain C++, the two routines of
the attention path whose arithmetic is not inside the external brotensor
library: ``build_axial_rope_tables`` (lines 116-184) and the softmax-attention
host loop of ``joint_attention_traced`` (lines 198-329).  That file is compiled
unmodified into ``oracle/_ref/libref.so`` (``oracle/Makefile``); its outputs on
small seeded inputs are committed as ``tests/golden/ref_pin.npz``
(``tests/golden/make_ref_pin.py``).  These tests hold the oracle restatement
to both: to the fixture everywhere, and to the library itself where it has
been built.  ``rms_norm_forward`` and ``rope_apply`` are brotensor operators and
stay unpinned; the attention cases therefore use identity rotation tables.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_ref_pin as pin  # noqa: E402

PIN = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_pin.npz")))


def oracle_case(oracle, name):
    txt, hp, wp, nh, hd, axes, with_bias = pin.CASES[name]
    cos, sin = oracle.flux_rope_tables(txt, hp, wp, hd, axes)
    q, k, v, bias = pin.inputs(name)
    out, avg = oracle.sdpa(q, k, v, nh, bias=bias, bias_row0=txt, want_avg=True)
    return cos, sin, out, avg


@pytest.mark.parametrize("name", sorted(pin.CASES))
def test_oracle_matches_reference_fixture(oracle, name):
    cos, sin, out, avg = oracle_case(oracle, name)
    # tables: same double-precision formula, rounded once to FP32
    np.testing.assert_array_equal(cos, PIN[f"{name}_cos"])
    np.testing.assert_array_equal(sin, PIN[f"{name}_sin"])
    # attention: same statement order (double scores, float P.V accumulation)
    # (one FP32 ulp: the oracle is built with fused multiply-add contraction)
    np.testing.assert_allclose(out, PIN[f"{name}_out"], rtol=0, atol=2.4e-7)
    np.testing.assert_array_equal(avg, PIN[f"{name}_avg"])
    assert np.allclose(PIN[f"{name}_avg"].sum(axis=1), 1.0, atol=1e-5)


def _ref():
    from oracle import ref
    if not ref.available():
        if not ref.can_build():
            pytest.skip("oracle/_ref is not built and the brodiffusion source tree is not on this host")
        ref.build()
    return ref


@pytest.mark.parametrize("name", sorted(pin.CASES))
def test_fixture_is_what_the_reference_computes(name):
    """The committed fixture equals a fresh run of the compiled reference file."""
    ref = _ref()
    txt, hp, wp, nh, hd, axes, with_bias = pin.CASES[name]
    cos, sin = ref.flux_rope_tables(txt, hp, wp, hd, axes)
    q, k, v, bias = pin.inputs(name)
    L = txt + hp * wp
    one, zero = np.ones((L, hd // 2), np.float32), np.zeros((L, hd // 2), np.float32)
    out, avg = ref.joint_attention_traced(q, k, v, one, zero, hd, nh, txt, bias)
    np.testing.assert_array_equal(cos, PIN[f"{name}_cos"])
    np.testing.assert_array_equal(sin, PIN[f"{name}_sin"])
    np.testing.assert_array_equal(out, PIN[f"{name}_out"])
    np.testing.assert_array_equal(avg, PIN[f"{name}_avg"])


def test_oracle_matches_reference_on_random_shapes(oracle):
    """Beyond the fixture: seeded shapes with odd text lengths, one to four heads,
    BF16-rounded inputs (the reference then returns a BF16-rounded output)."""
    ref = _ref()
    import synth
    rng = np.random.default_rng(77)
    for case in range(6):
        txt, hp, wp = int(rng.integers(0, 9)), int(rng.integers(1, 6)), int(rng.integers(1, 6))
        nh, hd = int(rng.integers(1, 5)), int(rng.choice([8, 16, 64]))
        axes = {8: (2, 2, 4), 16: (4, 6, 6), 64: (8, 28, 28)}[hd]
        L, D = txt + hp * wp, nh * hd
        q, k, v = (oracle.round_bf16(synth.activations((L, D), 500 + 10 * case + i)) for i in range(3))
        bias = synth.activations((hp * wp, txt), 505 + 10 * case) if txt > 0 and case % 2 == 0 else None
        c_ref, s_ref = ref.flux_rope_tables(txt, hp, wp, hd, axes)
        c_or, s_or = oracle.flux_rope_tables(txt, hp, wp, hd, axes)
        np.testing.assert_array_equal(c_or, c_ref)
        np.testing.assert_array_equal(s_or, s_ref)
        one, zero = np.ones((L, hd // 2), np.float32), np.zeros((L, hd // 2), np.float32)
        o_ref, a_ref = ref.joint_attention_traced(q, k, v, one, zero, hd, nh, txt, bias, bf16=True)
        o_or, a_or = oracle.sdpa(q, k, v, nh, bias=bias, bias_row0=txt, want_avg=True)
        np.testing.assert_allclose(oracle.round_bf16(o_or), o_ref, rtol=0, atol=2e-2)   # one BF16 ulp at |o| < 4
        assert np.abs(oracle.round_bf16(o_or) - o_ref).mean() < 1e-5
        np.testing.assert_allclose(a_or, a_ref, rtol=0, atol=1e-7)


def test_reference_error_messages():
    ref = _ref()
    with pytest.raises(RuntimeError, match="axes_dims_rope must sum to head_dim"):
        ref.flux_rope_tables(2, 2, 2, 8, (2, 2, 2))
    with pytest.raises(RuntimeError, match="head_dim must be even"):
        ref.flux_rope_tables(2, 2, 2, 7, (2, 2, 3))
