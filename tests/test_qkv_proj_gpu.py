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


def test_wide_tile_projection_matches_oracle(bd, oracle):
    """Large enough for the persistent 128 x 256-tile kernel: 18 row tiles x 4
    column tiles x 3 projections = 216 tiles (more than one per SM, so some CTAs
    walk two tiles and the stage ring and both accumulators wrap); two heads of
    128 per tile, five K blocks with a ragged last one."""
    rows, din, nh, hd = 2304 - 5, 296, 8, 128
    D = nh * hd
    x = synth.activations((rows, din), 9500)
    wq, wk, wv = (synth.round_bf16(synth.normal((D, din), 9501 + i, 0, 0.06)) for i in range(3))
    bk = synth.weights((D,), 9510)
    gq, gk = synth.gains(hd, 9511, "f32"), synth.gains(hd, 9512, "f32")
    cos, sin = oracle.flux_rope_tables(256, 48, 48, hd)      # 2560 table rows
    q = torch.full((rows, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    k, v = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
    bd.qkv_norm_rope_fwd(G.dev(x), G.dev(wq), G.dev(wk), G.dev(wv), q, k, v, nh, hd,
                         gain_q=G.dev(gq, torch.float32), gain_k=G.dev(gk, torch.float32),
                         cos=G.dev(cos, torch.float32), sin=G.dev(sin, torch.float32), rope_row0=3,
                         bk=G.dev(bk))
    assert bd.device_status() == 0
    rq = oracle.rope_apply(oracle.rms_norm_heads(oracle.linear(x, wq), nh, hd, gq), nh, hd, cos[3:], sin[3:])
    rk = oracle.rope_apply(oracle.rms_norm_heads(oracle.linear(x, wk, bk), nh, hd, gk), nh, hd, cos[3:], sin[3:])
    rv = oracle.linear(x, wv)
    assert np.abs(G.host(q) - rq).max() < 2.5e-2
    assert np.abs(G.host(k) - rk).max() < 2.5e-2
    G.check(G.host(v), rv, max_abs=2.5e-2, what="V projection (wide tiles)")


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("hd", [0, 64])
def test_wide_tile_linear_matches_oracle(bd, oracle, dtype, hd):
    """Plain linear layer (hd 0, 162 tiles) and four heads of 64 per tile
    (3 x 72 tiles), FP16 and BF16, bias, K not a multiple of 64."""
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    rnd = synth.round_bf16 if dtype == "bf16" else (lambda a: a.astype(np.float16).astype(np.float32))
    if hd == 0:
        rows, din, N = 2300, 200, 2304
        x = rnd(synth.normal((rows, din), 9600, 0, 1.0))
        w = rnd(synth.normal((N, din), 9601, 0, 0.06))
        b = rnd(synth.normal((N,), 9602, 0, 0.5))
        y = torch.full((rows, N), float("nan"), device="cuda", dtype=tdt)
        bd.linear_fwd(G.dev(x, tdt), G.dev(w, tdt), G.dev(b, tdt), y)
        assert bd.device_status() == 0
        G.check(G.host(y), oracle.linear(x, w, b), max_abs=2.5e-2, what="linear (wide tiles)")
    else:
        rows, din, nh = 2304, 136, 16
        D = nh * hd
        x = rnd(synth.normal((rows, din), 9610, 0, 1.0))
        ws = [rnd(synth.normal((D, din), 9611 + i, 0, 0.06)) for i in range(3)]
        g = synth.gains(hd, 9620, "f32")
        cos, sin = oracle.flux_rope_tables(256, 48, 48, hd, (8, 28, 28))
        outs = [torch.full((rows, D), float("nan"), device="cuda", dtype=tdt) for _ in range(3)]
        tg = G.dev(g, torch.float32)
        bd.qkv_norm_rope_fwd(G.dev(x, tdt), *[G.dev(w, tdt) for w in ws], *outs, nh, hd, gain_q=tg, gain_k=tg,
                             cos=G.dev(cos, torch.float32), sin=G.dev(sin, torch.float32))
        assert bd.device_status() == 0
        for i in range(3):
            ref = oracle.linear(x, ws[i])
            if i < 2:
                ref = oracle.rope_apply(oracle.rms_norm_heads(ref, nh, hd, g), nh, hd, cos, sin)
            assert np.abs(G.host(outs[i]) - ref).max() < 2.5e-2


def test_errors(bd):
    x = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(80, 64, device="cuda", dtype=torch.bfloat16)
    o = torch.zeros(8, 80, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_qkv_norm_rope_fwd: head_dim must be 64 or 128"):
        bd.qkv_norm_rope_fwd(x, w, w, w, o, o, o, 2, 40)
