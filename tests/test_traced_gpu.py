"""Traced / steered attention on the device against the oracle's statement of
dit::joint_attention_traced (src/dit/common.cpp:198-329): logit bias on the
image-query x text-key block and the head-averaged softmax block."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu


def test_golden_flux_tiny_bias_and_map(bd, golden):
    g = golden
    nh, hd, txt = 2, 8, 3
    q, k, v = G.dev(g["flux_q"]), G.dev(g["flux_k"]), G.dev(g["flux_v"])
    cos, sin = G.dev(g["flux_cos"], torch.float32), G.dev(g["flux_sin"], torch.float32)
    qr, kr = torch.empty_like(q), torch.empty_like(k)
    bd.rmsnorm_rope([dict(x=q, out=qr, gain=G.dev(g["flux_gq"]), cos=cos, sin=sin),
                     dict(x=k, out=kr, gain=G.dev(g["flux_gk"]), cos=cos, sin=sin)], nh, hd)
    L = q.shape[0]
    out = torch.empty_like(q)
    amap = bd.sdpa_traced_fwd(qr, kr, v, out, nh, map_row0=0, map_rows=L, map_cols=L)
    assert bd.device_status() == 0
    G.check(G.host(out), g["flux_out"], what="traced output")
    assert np.abs(G.host(amap) - g["flux_avg"]).max() < 2e-2
    # rows of the full map are non-negative and sum to one (tests/test_flux_blocks.cpp:268-281)
    m = G.host(amap)
    assert m.min() >= 0.0 and np.abs(m.sum(1) - 1.0).max() < 2e-2
    outb = torch.empty_like(q)
    bd.sdpa_traced_fwd(qr, kr, v, outb, nh, bias=G.dev(g["flux_bias"], torch.float32), bias_row0=txt)
    assert bd.device_status() == 0
    G.check(G.host(outb), g["flux_out_biased"], what="biased output")


def test_flux_image_to_text_block(bd, oracle):
    """The block Flux keeps: image-query rows x text-key columns, with a bias that
    steers image tokens toward some text tokens (tests/test_flux_blocks.cpp:343-386)."""
    nh, hd, txt, img = 4, 128, 96, 400
    L, D = txt + img, nh * hd
    q, k, v = (synth.activations((L, D), 9100 + i) for i in range(3))
    bias = np.zeros((img, txt), np.float32)
    bias[:, 10:20] = 2.0
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    out = torch.empty_like(tq)
    amap = bd.sdpa_traced_fwd([tq[:txt], tq[txt:]], [tk[:txt], tk[txt:]], [tv[:txt], tv[txt:]],
                              [out[:txt], out[txt:]], nh, bias=G.dev(bias, torch.float32), bias_row0=txt,
                              map_row0=txt, map_rows=img, map_cols=txt)
    assert bd.device_status() == 0
    ref_out, ref_avg = oracle.sdpa(q, k, v, nh, bias=bias, bias_row0=txt, want_avg=True)
    G.check(G.host(out), ref_out, what="steered output")
    got = G.host(amap)
    assert np.abs(got - ref_avg[txt:, :txt]).max() < 5e-3
    # steering is monotone: biased columns receive more weight than without bias
    amap0 = bd.sdpa_traced_fwd(tq, tk, tv, torch.empty_like(tq), nh, map_row0=txt, map_rows=img, map_cols=txt)
    assert G.host(amap)[:, 10:20].sum() > G.host(amap0)[:, 10:20].sum()


def test_unet_cross_attention_map(bd, oracle):
    """U-Net trace mode: map (Lq, 77) over all rows with a full (Lq, Lk) logit
    bias; rows sum to one within 0.05 (tests/test_unet.cpp:487-500)."""
    nh, hd, Lq, Lk = 8, 40, 256, 77
    q = synth.activations((Lq, nh * hd), 9201)
    k = synth.activations((Lk, nh * hd), 9202)
    v = synth.activations((Lk, nh * hd), 9203)
    bias = synth.normal((Lq, Lk), 9204, 0, 0.5)
    out = torch.empty(Lq, nh * hd, device="cuda", dtype=torch.bfloat16)
    amap = bd.sdpa_traced_fwd(G.dev(q), G.dev(k), G.dev(v), out, nh, bias=G.dev(bias, torch.float32),
                              map_rows=Lq, map_cols=Lk)
    assert bd.device_status() == 0
    ref_out, ref_avg = oracle.sdpa(q, k, v, nh, bias=bias, want_avg=True)
    G.check(G.host(out), ref_out, what="unet traced output")
    got = G.host(amap)
    assert np.abs(got - ref_avg).max() < 5e-3
    assert np.abs(got.sum(1) - 1.0).max() < 0.05


def test_map_agrees_with_masked_attention(bd, oracle):
    """The map block follows the visibility rules the attention itself used: a
    masked or future key has weight 0 and every visible row still sums to one."""
    nh, hd, Lq, Lk = 4, 64, 200, 200
    q, k, v = (synth.activations((Lq, nh * hd), 9300 + i) for i in range(3))
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    # key mask (padded caption tail + a hole)
    mask = np.ones(Lk, np.float32)
    mask[150:] = 0.0
    mask[7] = 0.0
    out = torch.empty_like(tq)
    amap = bd.sdpa_traced_fwd(tq, tk, tv, out, nh, map_rows=Lq, map_cols=Lk, key_mask=G.dev(mask, torch.float32))
    assert bd.device_status() == 0
    ref_out, ref_avg = oracle.sdpa(q, k, v, nh, key_mask=mask, want_avg=True)
    G.check(G.host(out), ref_out, what="key-masked traced output")
    m = G.host(amap)
    assert np.abs(m - ref_avg).max() < 5e-3
    assert np.all(m[:, mask == 0.0] == 0.0)
    assert np.abs(m.sum(1) - 1.0).max() < 2e-2
    # causal
    out_c = torch.empty_like(tq)
    amap_c = bd.sdpa_traced_fwd(tq, tk, tv, out_c, nh, map_rows=Lq, map_cols=Lk, mask_mode=bd.MASK_CAUSAL)
    assert bd.device_status() == 0
    ref_out_c, ref_avg_c = oracle.sdpa(q, k, v, nh, mask_mode=1, want_avg=True)
    G.check(G.host(out_c), ref_out_c, what="causal traced output")
    mc = G.host(amap_c)
    assert np.abs(mc - ref_avg_c).max() < 5e-3
    assert np.all(np.triu(mc, 1) == 0.0)
    assert mc.max() <= 1.0 + 1e-3 and np.abs(mc.sum(1) - 1.0).max() < 2e-2


def test_errors(bd):
    q = torch.zeros(64, 256, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(100, 10, device="cuda")
    with pytest.raises(bd.BdattnError, match=r"^joint_attention_traced: bias block"):
        bd.sdpa_traced_fwd(q, q, q, q.clone(), 2, bias=b)
