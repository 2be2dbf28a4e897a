"""Q/K/V projection with per-head RMSNorm + RoPE fused into the GEMM epilogue,
against the oracle's linear -> rms_norm_heads -> rope_apply."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,din,nh,hd", [(300, 256, 4, 128), (130, 192, 6, 64), (1, 64, 1, 128)])
def test_qkv_norm_rope_matches_oracle(bd, oracle, rows, din, nh, hd):
    D = nh * hd
    x = synth.activations((rows, din), 9300 + rows)
    wq, wk, wv = (synth.round_bf16(synth.normal((D, din), 9301 + rows + i, 0, 0.06)) for i in range(3))
    bq = synth.weights((D,), 9310 + rows)
    gq, gk = synth.gains(hd, 9311 + rows, "f32"), synth.gains(hd, 9312 + rows, "f32")
    axes = (16, 56, 56) if hd == 128 else (8, 28, 28)
    row0 = 7
    cos, sin = oracle.flux_rope_tables(4, 20, 20, hd, axes)     # 404 table rows >= row0 + rows
    q = torch.full((rows, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    k, v = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
    bd.qkv_norm_rope_fwd(G.dev(x), G.dev(wq), G.dev(wk), G.dev(wv), q, k, v, nh, hd,
                         gain_q=G.dev(gq, torch.float32), gain_k=G.dev(gk, torch.float32),
                         cos=G.dev(cos, torch.float32), sin=G.dev(sin, torch.float32), rope_row0=row0,
                         bq=G.dev(bq))
    assert bd.device_status() == 0
    rq = oracle.rope_apply(oracle.rms_norm_heads(oracle.linear(x, wq, bq), nh, hd, gq), nh, hd,
                           cos[row0:], sin[row0:])
    rk = oracle.rope_apply(oracle.rms_norm_heads(oracle.linear(x, wk), nh, hd, gk), nh, hd,
                           cos[row0:], sin[row0:])
    rv = oracle.linear(x, wv)
    # one BF16 rounding of values up to ~5
    assert np.abs(G.host(q) - rq).max() < 2.5e-2
    assert np.abs(G.host(k) - rk).max() < 2.5e-2
    G.check(G.host(v), rv, max_abs=2.5e-2, what="V projection")


def test_fused_projection_feeds_attention(bd, oracle):
    """Projection -> attention, the Flux single-stream attention sublayer."""
    rows, din, nh, hd = 384, 256, 2, 128
    D = nh * hd
    x = synth.activations((rows, din), 9401)
    wq, wk, wv = (synth.round_bf16(synth.normal((D, din), 9402 + i, 0, 0.06)) for i in range(3))
    g = synth.gains(hd, 9410, "f32")
    cos, sin = oracle.flux_rope_tables(128, 16, 16, hd)
    q = torch.empty(rows, D, device="cuda", dtype=torch.bfloat16)
    k, v, out = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    tg = G.dev(g, torch.float32)
    bd.qkv_norm_rope_fwd(G.dev(x), G.dev(wq), G.dev(wk), G.dev(wv), q, k, v, nh, hd, gain_q=tg, gain_k=tg,
                         cos=G.dev(cos, torch.float32), sin=G.dev(sin, torch.float32))
    bd.sdpa_fwd(q, k, v, out, nh)
    assert bd.device_status() == 0
    rq = oracle.rope_apply(oracle.rms_norm_heads(oracle.linear(x, wq), nh, hd, g), nh, hd, cos, sin)
    rk = oracle.rope_apply(oracle.rms_norm_heads(oracle.linear(x, wk), nh, hd, g), nh, hd, cos, sin)
    ref = oracle.sdpa(rq, rk, oracle.linear(x, wv), nh)
    G.check(G.host(out), ref, max_abs=3e-2, what="projection + attention")


def test_errors(bd):
    x = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(80, 64, device="cuda", dtype=torch.bfloat16)
    o = torch.zeros(8, 80, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_qkv_norm_rope_fwd: head_dim must be 64 or 128"):
        bd.qkv_norm_rope_fwd(x, w, w, w, o, o, o, 2, 40)
