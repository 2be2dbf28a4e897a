"""Generates tests/golden/golden.npz.

The expected outputs are computed with PyTorch in float64 on the CPU,
written directly from the formulas of the reference (cited per case) and
independently of the oracle under oracle/: the fixtures pin the oracle, and
the CUDA path is then checked against both.  Inputs come from tests/synth.py
and are stored in the file, so the fixtures do not depend on the generator.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import synth  # noqa: E402

T = torch.float64


def bits(x):
    """BF16 bit patterns of an array of exactly-BF16 float32 values."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def t(x):
    return torch.from_numpy(np.asarray(x)).to(T)


def axial_tables(positions, axes, theta):
    """positions: (L, n_axes) ints.  cos/sin (L, sum(axes)/2): axis a owns
    axes[a]/2 consecutive pairs with omega = theta^(-2p/axes[a])
    (src/dit/common.cpp:147-158, src/dit/qwenimage21_forward.cpp:171-196)."""
    cols = []
    for a, d in enumerate(axes):
        p = torch.arange(d // 2, dtype=T)
        omega = torch.pow(torch.tensor(theta, dtype=T), -2.0 * p / d)
        cols.append(t(positions[:, a])[:, None] * omega[None, :])
    ang = torch.cat(cols, dim=1)
    return torch.cos(ang).float().numpy(), torch.sin(ang).float().numpy()


def flux_positions(txt_len, hp, wp):
    pos = [(0, 0, 0)] * txt_len
    pos += [(0, i, j) for i in range(hp) for j in range(wp)]
    return np.asarray(pos, np.int64)


def qwen_positions(prefix, hp, wp):
    """src/dit/qwenimage21_forward.cpp:136-165."""
    pos, p = [], 0
    def image(h, w, p):
        h0, w0 = -(h - h // 2), -(w - w // 2)
        return [(p, h0 + i, w0 + j) for i in range(h) for j in range(w)], p + max(h, w)
    for s in prefix:
        if s[0] == "text":
            pos += [(p + i,) * 3 for i in range(s[1])]
            p += s[1]
        else:
            blk, p = image(s[1], s[2], p)
            pos += blk
    blk, p = image(hp, wp, p)
    pos += blk
    return np.asarray(pos, np.int64)


def rms_heads(x, nh, hd, gain, eps):
    L = x.shape[0]
    xv = t(x).view(L, nh, hd)
    y = xv * torch.rsqrt((xv * xv).mean(-1, keepdim=True) + eps) * t(gain)
    return y.reshape(L, nh * hd)


def rope(x, nh, hd, cos, sin, pair_mode=0):
    L = x.shape[0]
    xv = x.view(L, nh, hd)
    c, s = t(cos)[:, None, :], t(sin)[:, None, :]
    if pair_mode == 0:
        a, b = xv[..., 0::2], xv[..., 1::2]
        out = torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(L, nh, hd)
    else:
        a, b = xv[..., : hd // 2], xv[..., hd // 2:]
        out = torch.cat([a * c - b * s, a * s + b * c], dim=-1)
    return out.reshape(L, nh * hd)


def attention(q, k, v, nh, mask=None, bias=None):
    """softmax(q k^T / sqrt(hd) + bias [mask]) v per head; rows with no
    visible key give 0 (src/dit/common.cpp:246-305)."""
    Lq, D = q.shape
    Lk = k.shape[0]
    hd = D // nh
    qh = q.view(Lq, nh, hd).transpose(0, 1)
    kh = k.view(Lk, nh, hd).transpose(0, 1)
    vh = v.view(Lk, nh, hd).transpose(0, 1)
    s = qh @ kh.transpose(1, 2) / math.sqrt(hd)
    if bias is not None:
        s = s + bias
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.max(-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    p = torch.where(den > 0, e / den, torch.zeros_like(e))
    return (p @ vh).transpose(0, 1).reshape(Lq, D), p.mean(0)


def main():
    out = {}
    # --- tiny Flux joint attention: the reference's synthetic config
    # (tests/test_flux_blocks.cpp:480-507): 2 heads x 8, axes {2,2,4},
    # txt_len 3, 4x4 packed latent.
    nh, hd, txt, hp, wp = 2, 8, 3, 4, 4
    L = txt + hp * wp
    cos, sin = axial_tables(flux_positions(txt, hp, wp), (2, 2, 4), 10000.0)
    q = synth.activations((L, nh * hd), 101)
    k = synth.activations((L, nh * hd), 102)
    v = synth.activations((L, nh * hd), 103)
    gq, gk = synth.gains(hd, 104), synth.gains(hd, 105)
    qn, kn = rms_heads(q, nh, hd, gq, 1e-6), rms_heads(k, nh, hd, gk, 1e-6)
    o, avg = attention(rope(qn, nh, hd, cos, sin), rope(kn, nh, hd, cos, sin), t(v), nh)
    bias = synth.normal((hp * wp, txt), 106)
    fb = torch.zeros(L, L, dtype=T)
    fb[txt:, :txt] = t(bias)
    ob, _ = attention(rope(qn, nh, hd, cos, sin), rope(kn, nh, hd, cos, sin), t(v), nh, bias=fb)
    out.update(flux_q=q, flux_k=k, flux_v=v, flux_gq=gq, flux_gk=gk, flux_cos=cos, flux_sin=sin,
               flux_qn=qn.float().numpy(), flux_qr=rope(qn, nh, hd, cos, sin).float().numpy(),
               flux_out=o.float().numpy(), flux_avg=avg.float().numpy(), flux_bias=bias,
               flux_out_biased=ob.float().numpy())

    # --- tiny Qwen-Image block-causal prefill: 2 heads x 64, axes {8,28,28}
    # (tests/qwenimage21_fixture.h:89-103); prefix = text 5 + image 2x3 +
    # text 4, target 4x4.  Key j visible to query i iff j <= i or both in the
    # same image segment (include/brodiffusion/dit/qwenimage21.h:31-33).
    nh, hd = 2, 64
    prefix = [("text", 5), ("image", 2, 3), ("text", 4)]
    hp, wp = 4, 4
    pos = qwen_positions(prefix, hp, wp)
    L = pos.shape[0]
    cos, sin = axial_tables(pos, (8, 28, 28), 10000.0)
    seg = []
    for i, s in enumerate(prefix + [("image", hp, wp)]):
        n = s[1] if s[0] == "text" else s[1] * s[2]
        seg += [(i, s[0] == "image")] * n
    ii = torch.arange(L)
    mask = ii[None, :] <= ii[:, None]
    for a in range(L):
        for b in range(L):
            if seg[a][0] == seg[b][0] and seg[a][1]:
                mask[a, b] = True
    q = synth.activations((L, nh * hd), 201)
    k = synth.activations((L, nh * hd), 202)
    v = synth.activations((L, nh * hd), 203)
    gq, gk = synth.gains(hd, 204, "f32"), synth.gains(hd, 205, "f32")
    qr = rope(rms_heads(q, nh, hd, gq, 1e-6), nh, hd, cos, sin)
    kr = rope(rms_heads(k, nh, hd, gk, 1e-6), nh, hd, cos, sin)
    o, _ = attention(qr, kr, t(v), nh, mask=mask)
    out.update(qwen_q=q, qwen_k=k, qwen_v=v, qwen_gq=gq, qwen_gk=gk, qwen_cos=cos, qwen_sin=sin,
               qwen_pos=pos.astype(np.int32), qwen_mask=mask.numpy(), qwen_out=o.float().numpy(),
               qwen_kr=kr.float().numpy())

    # --- head_dim 128 with key mask and q-offset causal (Lq 70, Lk 200)
    nh, hd, Lq, Lk = 2, 128, 40, 150
    q = synth.activations((Lq, nh * hd), 301)
    k = synth.activations((Lk, nh * hd), 302)
    v = synth.activations((Lk, nh * hd), 303)
    km = (synth.uniform01(Lk, 304) > 0.2).astype(np.float32)
    causal = torch.arange(Lk)[None, :] <= torch.arange(Lq)[:, None] + (Lk - Lq)
    o1, _ = attention(t(q), t(k), t(v), nh, mask=causal)
    o2, _ = attention(t(q), t(k), t(v), nh, mask=torch.from_numpy(km > 0)[None, :].expand(Lq, Lk))
    # inputs are exact BF16 values: stored as their 16-bit patterns
    out.update(hd128_q_bf16=bits(q), hd128_k_bf16=bits(k), hd128_v_bf16=bits(v), hd128_keymask=km,
               hd128_out_causal=o1.float().numpy(), hd128_out_keymask=o2.float().numpy())

    # --- SD1.5 self / cross attention block (src/unet_blocks.cpp:264-271,
    # 320-327): bias-less Q/K/V projections, biased output projection.
    nh, hd, Lx, Lc, Cc = 4, 8, 24, 7, 48
    C_ = nh * hd
    x = synth.activations((Lx, C_), 401, "f32")
    ctx = synth.activations((Lc, Cc), 402, "f32")
    wq, wk, wv, wo = (synth.normal((C_, C_), s, 0, 0.2) for s in (403, 404, 405, 406))
    wk2, wv2 = synth.normal((C_, Cc), 407, 0, 0.2), synth.normal((C_, Cc), 408, 0, 0.2)
    bo = synth.normal((C_,), 409, 0, 0.1)
    o, _ = attention(t(x) @ t(wq).T, t(x) @ t(wk).T, t(x) @ t(wv).T, nh)
    self_out = o @ t(wo).T + t(bo)
    o, _ = attention(t(x) @ t(wq).T, t(ctx) @ t(wk2).T, t(ctx) @ t(wv2).T, nh)
    cross_out = o @ t(wo).T + t(bo)
    out.update(sd_x=x, sd_ctx=ctx, sd_wq=wq, sd_wk=wk, sd_wv=wv, sd_wo=wo, sd_wk2=wk2, sd_wv2=wv2,
               sd_bo=bo, sd_self_out=self_out.float().numpy(), sd_cross_out=cross_out.float().numpy())

    # --- Sana ReLU linear attention (src/dit/sana.cpp:470-520), channel-major.
    nh, hd, N = 2, 32, 40
    q = synth.activations((nh * hd, N), 501)
    k = synth.activations((nh * hd, N), 502)
    v = synth.activations((nh * hd, N), 503)
    rq, rk = torch.relu(t(q)), torch.relu(t(k))
    o = torch.zeros(nh * hd, N, dtype=T)
    sz = torch.zeros(nh, hd + 1, hd, dtype=T)
    for h in range(nh):
        sl = slice(h * hd, (h + 1) * hd)
        S = t(v)[sl] @ rk[sl].T
        z = rk[sl].sum(1)
        sz[h, :hd], sz[h, hd] = S, z
        o[sl] = (S @ rq[sl]) / (z @ rq[sl] + 1e-15)
    out.update(sana_q=q, sana_k=k, sana_v=v, sana_out=o.float().numpy(), sana_sz=sz.float().numpy())

    # --- fused FF1 + exact GEGLU (src/fused_transformer.cu:89-92,275-282),
    # the reference test shape B40 64->48 (tests/test_fused_parity.cpp:268).
    B, Din, Dout = 40, 64, 48
    x = synth.activations((B, Din), 601, "fp16")
    w = synth.round_fp16(synth.normal((2 * Dout, Din), 602, 0, 0.1))
    b = synth.round_fp16(synth.normal((2 * Dout,), 603, 0, 0.2))
    tt = t(x) @ t(w).T + t(b)
    y = tt[:, :Dout] * torch.nn.functional.gelu(tt[:, Dout:], approximate="none")
    out.update(geglu_x=x, geglu_w=w, geglu_b=b, geglu_y=y.float().numpy())

    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {os.path.getsize(path)} bytes, {len(out)} arrays")


if __name__ == "__main__":
    main()
