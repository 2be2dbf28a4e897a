"""Softmax-attention parity on the GPU: the CUDA path, called through the C
ABI, against the golden fixtures and the CPU oracle on the same seeded inputs.
Tolerance of the path: BF16 GPU vs FP32 CPU oracle, max-abs
error <= 2e-2 after the output projection and cosine similarity >= 0.9999."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth
from conftest import bf16_from_bits

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ golden
def test_golden_hd128_causal_and_key_mask(bd, golden):
    g = golden
    q, k, v = (bf16_from_bits(g[f"hd128_{n}_bf16"]) for n in "qkv")
    o = G.sdpa(bd, q, k, v, 2, mask_mode=bd.MASK_CAUSAL)
    G.check(o, g["hd128_out_causal"], what="causal")
    o = G.sdpa(bd, q, k, v, 2, key_mask=g["hd128_keymask"])
    G.check(o, g["hd128_out_keymask"], what="key mask")


def test_golden_flux_tiny_joint_attention(bd, golden):
    """Reference tiny-Flux config (tests/test_flux_blocks.cpp:480-507): 2 heads
    x 8, norm + rope + attention through the C ABI."""
    g = golden
    q, k, v = G.dev(g["flux_q"]), G.dev(g["flux_k"]), G.dev(g["flux_v"])
    cos, sin = G.dev(g["flux_cos"], torch.float32), G.dev(g["flux_sin"], torch.float32)
    qr, kr = torch.empty_like(q), torch.empty_like(k)
    bd.rmsnorm_rope([dict(x=q, out=qr, gain=G.dev(g["flux_gq"]), cos=cos, sin=sin),
                     dict(x=k, out=kr, gain=G.dev(g["flux_gk"]), cos=cos, sin=sin)], 2, 8)
    out = torch.empty_like(q)
    bd.sdpa_fwd(qr, kr, v, out, 2)
    assert bd.device_status() == 0
    G.check(G.host(out), g["flux_out"], what="flux tiny")


def test_golden_qwen_block_causal_prefill_and_cached_step(bd, golden, oracle):
    """Prefill as per-segment calls (src/dit/qwenimage21_forward.cpp:650-676)
    and the cached step with two key/value segments (prefix cache + fresh
    rows), both against the golden block-causal output."""
    g = golden
    nh, hd = 2, 64
    q, k, v = G.dev(g["qwen_q"]), G.dev(g["qwen_k"]), G.dev(g["qwen_v"])
    cos, sin = G.dev(g["qwen_cos"], torch.float32), G.dev(g["qwen_sin"], torch.float32)
    qr, kr = torch.empty_like(q), torch.empty_like(k)
    bd.rmsnorm_rope([dict(x=q, out=qr, gain=G.dev(g["qwen_gq"], torch.float32), cos=cos, sin=sin),
                     dict(x=k, out=kr, gain=G.dev(g["qwen_gk"], torch.float32), cos=cos, sin=sin)],
                    nh, hd)
    G.check(G.host(kr), g["qwen_kr"], max_abs=3e-2, what="post-rope K")
    out = torch.full_like(q, float("nan"))
    start = 0
    for kind, n in (("text", 5), ("image", 6), ("text", 4)):
        end = start + n
        bd.sdpa_fwd(qr[start:end], kr[:end], v[:end], out[start:end], nh,
                    mask_mode=bd.MASK_CAUSAL if kind == "text" else bd.MASK_NONE)
        start = end
    bd.sdpa_fwd(qr[start:], kr, v, out[start:], nh)
    assert bd.device_status() == 0
    G.check(G.host(out), g["qwen_out"], what="prefill")
    # cached step: prefix K/V snapshot (own buffers) + fresh target rows
    ck, cv = kr[:start].clone(), v[:start].clone()
    out_c = torch.full_like(q[start:], float("nan"))
    bd.sdpa_fwd(qr[start:], [ck, kr[start:]], [cv, v[start:]], out_c, nh)
    assert bd.device_status() == 0
    G.check(G.host(out_c), g["qwen_out"][start:], what="cached step")
    # cached vs prefill (tests/test_qwenimage21_dit.cpp:117-128 bounds the FP32
    # CPU paths by 2e-3 relative); the key tiles are cut differently in the
    # two calls, so BF16 outputs may differ in the last place: the reference's
    # BF16 bound of 1e-2 (tests/test_flux_blocks.cpp:283-300) applies
    G.check(G.host(out_c), G.host(out[start:]), max_abs=1e-2, what="cached vs prefill")


# ------------------------------------------------------- config-shaped cases
def _flux_case(L_txt, hp, wp, nh=24, hd=128, seed=2000):
    L = L_txt + hp * wp
    D = nh * hd
    q = synth.activations((L, D), seed + 1)
    k = synth.activations((L, D), seed + 2)
    v = synth.activations((L, D), seed + 3)
    return L, D, q, k, v


def test_flux_1024_joint_attention_full_size(bd, oracle):
    """Flux.1 at 1024 px: 512 text + 4096 image tokens, 24 heads x 128, per-head QK
    RMSNorm, 3-axis RoPE (16,56,56), double-stream (text and image given as
    separate segments with separate gains) and single-stream variants."""
    nh, hd, txt, hp, wp = 24, 128, 512, 64, 64
    L, D, q, k, v = _flux_case(txt, hp, wp)
    g = [synth.gains(hd, 2010 + i) for i in range(4)]       # norm_q, norm_k, norm_added_q, norm_added_k
    cos, sin = oracle.flux_rope_tables(txt, hp, wp, hd)
    wo = synth.weights((D, D), 2020)
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    tcos, tsin = G.dev(cos, torch.float32), G.dev(sin, torch.float32)
    # double-stream: text rows use the added_* gains, image rows norm_q/norm_k
    qr, kr = torch.empty_like(tq), torch.empty_like(tk)
    bd.rmsnorm_rope([
        dict(x=tq[:txt], out=qr[:txt], gain=G.dev(g[2]), cos=tcos, sin=tsin, rope_row0=0),
        dict(x=tq[txt:], out=qr[txt:], gain=G.dev(g[0]), cos=tcos, sin=tsin, rope_row0=txt),
        dict(x=tk[:txt], out=kr[:txt], gain=G.dev(g[3]), cos=tcos, sin=tsin, rope_row0=0),
        dict(x=tk[txt:], out=kr[txt:], gain=G.dev(g[1]), cos=tcos, sin=tsin, rope_row0=txt),
    ], nh, hd)
    out = torch.full_like(tq, float("nan"))
    bd.sdpa_fwd([qr[:txt], qr[txt:]], [kr[:txt], kr[txt:]], [tv[:txt], tv[txt:]],
                [out[:txt], out[txt:]], nh)
    assert bd.device_status() == 0
    # single launch over the unsplit tensors gives the same bits
    out1 = torch.full_like(tq, float("nan"))
    bd.sdpa_fwd(qr, kr, tv, out1, nh)
    out2 = torch.full_like(tq, float("nan"))
    bd.sdpa_fwd(qr, kr, tv, out2, nh)
    assert bd.device_status() == 0
    assert torch.equal(out1, out2), "two runs differ"
    assert torch.equal(out, out1), "segmented and unsegmented results differ"

    # oracle on sampled query rows (all heads, all keys)
    def norm(x, gt, gi):
        return np.concatenate([oracle.rms_norm_heads(x[:txt], nh, hd, gt),
                               oracle.rms_norm_heads(x[txt:], nh, hd, gi)])
    qn, kn = norm(q, g[2], g[0]), norm(k, g[3], g[1])
    qro = oracle.rope_apply(qn, nh, hd, cos, sin)
    kro = oracle.rope_apply(kn, nh, hd, cos, sin)
    rows = G.boundary_rows(L)
    ref = oracle.sdpa(qro, kro, v, nh, rows=rows)
    got = G.host(out)[rows]
    err, cosv = G.check(got, ref, what="flux1024 attention output")
    # after the output projection (north-star gate)
    G.check(got @ wo.T, ref @ wo.T, what="flux1024 after out-projection")
    # softmax output is a convex combination of V rows
    vmax = np.abs(v).max()
    assert np.abs(G.host(out)).max() <= vmax + 1e-2


def test_flux_single_stream_output_into_wider_rows(bd, oracle):
    """Single-stream variant writes attention straight into the (L, 5D)
    concatenation buffer (src/dit/flux.cpp:626-632) through o_ld."""
    nh, hd, L = 4, 128, 300
    D = nh * hd
    q, k, v = (synth.activations((L, D), 2100 + i) for i in range(3))
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    cat5 = torch.zeros(L, 5 * D, device="cuda", dtype=torch.bfloat16)
    bd.sdpa_fwd(tq, tk, tv, cat5[:, :D], nh)
    assert bd.device_status() == 0
    G.check(G.host(cat5[:, :D]), oracle.sdpa(q, k, v, nh), what="cat5 layout")
    assert torch.count_nonzero(cat5[:, D:]) == 0


def test_qwen_cached_step_full_size(bd, oracle):
    """Qwen-Image cached step: 256 cached prefix rows + 4096 fresh rows, 24 x 128; prefix
    K/V come from their own buffers (no k_full_/v_full_ copy)."""
    nh, hd, P, T = 24, 128, 256, 4096
    D = nh * hd
    q = synth.activations((T, D), 3001)
    k = synth.activations((P + T, D), 3002)
    v = synth.activations((P + T, D), 3003)
    wo = synth.weights((D, D), 3004)
    rows = G.boundary_rows(T)
    out = G.sdpa(bd, q, [k[:P], k[P:]], [v[:P], v[P:]], nh)
    ref = oracle.sdpa(q, k, v, nh, rows=rows)
    G.check(out[rows], ref, what="qwen cached")
    G.check(out[rows] @ wo.T, ref @ wo.T, what="qwen cached after out-projection")
    # prefix attenuation hook (src/dit/qwenimage21_forward.cpp:606-645)
    ks = np.ones(P + T, np.float32); ks[:P] = 0.5
    vs = np.ones(P + T, np.float32); vs[:P] = 0.25
    out_s = G.sdpa(bd, q, [k[:P], k[P:]], [v[:P], v[P:]], nh, key_scale=ks, val_scale=vs)
    ref_s = oracle.sdpa(q, k * ks[:, None], v * vs[:, None], nh, rows=rows[:8])
    G.check(out_s[rows[:8]], ref_s, what="prefix K/V scale")


def test_qwen_extract_step_text_prefix(bd, oracle):
    """Qwen-Image step 0: text prefix of 256 rows attends causally (one run of
    256 == four blocks of 64), target rows attend everything."""
    nh, hd, P, T = 24, 128, 256, 1024
    D = nh * hd
    q = synth.activations((P + T, D), 3101)
    k = synth.activations((P + T, D), 3102)
    v = synth.activations((P + T, D), 3103)
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    out = torch.full_like(tq, float("nan"))
    bd.sdpa_fwd(tq[:P], tk[:P], tv[:P], out[:P], nh, mask_mode=bd.MASK_CAUSAL)
    bd.sdpa_fwd(tq[P:], tk, tv, out[P:], nh)
    assert bd.device_status() == 0
    seg_id, is_img = oracle.block_causal_tables([("text", P), ("image", T)])
    rows = np.concatenate([G.boundary_rows(P, extra=8), P + G.boundary_rows(T, extra=8)])
    ref = oracle.sdpa(q, k, v, nh, mask_mode=2, seg_id=seg_id, seg_is_image=is_img, rows=rows)
    G.check(G.host(out)[rows], ref, what="qwen extract")
    # four causal blocks of 64 with growing key ranges give the same bits
    out4 = torch.full_like(tq[:P], float("nan"))
    for s in range(0, P, 64):
        bd.sdpa_fwd(tq[s:s + 64], tk[:s + 64], tv[:s + 64], out4[s:s + 64], nh,
                    mask_mode=bd.MASK_CAUSAL)
    assert bd.device_status() == 0
    G.check(G.host(out4), G.host(out[:P]), max_abs=1e-2, what="4x64 blocks vs one run")


def test_qwen_extract_step_image_prefix_segments(bd, oracle):
    """Step 0 with a prefix of four condition images of 8 x 8 tokens
    (block-bidirectional: each sees itself and everything before it) ahead of
    the target rows, at the model width (24 heads x 128).  The whole layer path
    runs on the device the way src/dit/qwenimage21_forward.cpp:579-676 runs it:
    RoPE rows from the running-position rule, per-head RMSNorm with FP32 gains +
    RoPE, then one unmasked call per image segment over K[0:end) and one call for
    the target rows over every key (src/dit/qwenimage21_forward.cpp:650-676; rule
    in include/brodiffusion/dit/qwenimage21.h:31-33)."""
    nh, hd, hp, wp = 24, 128, 32, 32
    prefix = [("image", 8, 8)] * 4
    P, T = 4 * 64, hp * wp
    L, D = P + T, nh * hd
    q = synth.activations((L, D), 3201)
    k = synth.activations((L, D), 3202)
    v = synth.activations((L, D), 3203)
    gq, gk = synth.gains(hd, 3204), synth.gains(hd, 3205)
    wo = synth.weights((D, D), 3206)
    cos, sin = bd.rope_tables_qwen(prefix, hp, wp, hd)
    assert cos.shape == (L, hd // 2)
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    qr, kr = torch.empty_like(tq), torch.empty_like(tk)
    bd.rmsnorm_rope([dict(x=tq, out=qr, gain=G.dev(gq, torch.float32), cos=cos, sin=sin),
                     dict(x=tk, out=kr, gain=G.dev(gk, torch.float32), cos=cos, sin=sin)], nh, hd)
    out = torch.full_like(tq, float("nan"))
    start = 0
    for _, h, w in prefix:
        end = start + h * w
        bd.sdpa_fwd(qr[start:end], kr[:end], tv[:end], out[start:end], nh)     # unmasked over [0, end)
        start = end
    bd.sdpa_fwd(qr[start:], kr, tv, out[start:], nh)
    assert bd.device_status() == 0
    # oracle: the block-causal rule stated directly on the whole sequence
    rc, rs = oracle.qwen_rope_tables(prefix, hp, wp, hd)
    qo = oracle.rope_apply(oracle.rms_norm_heads(oracle.round_bf16(q), nh, hd, gq), nh, hd, rc, rs)
    ko = oracle.rope_apply(oracle.rms_norm_heads(oracle.round_bf16(k), nh, hd, gk), nh, hd, rc, rs)
    seg_id, is_img = oracle.block_causal_tables([("image", 64)] * 4 + [("image", T)])
    # every prefix row (all four blocks and their edges) + sampled target rows
    rows = np.concatenate([np.arange(P, dtype=np.int32), P + G.boundary_rows(T, extra=8)])
    ref = oracle.sdpa(qo, ko, oracle.round_bf16(v), nh, mask_mode=2, seg_id=seg_id, seg_is_image=is_img, rows=rows)
    got = G.host(out)[rows]
    G.check(got, ref, what="qwen image-segment prefill")
    G.check(got @ wo.T, ref @ wo.T, what="qwen image-segment prefill after out-projection")
    # a row of block b must not see block b + 1: move a later block's V and the
    # earlier rows' output is unchanged bit for bit
    tv2 = tv.clone()
    tv2[192:256] += 1.0
    out2 = torch.full_like(out[:192], float("nan"))
    start = 0
    for _ in range(3):
        bd.sdpa_fwd(qr[start:start + 64], kr[:start + 64], tv2[:start + 64], out2[start:start + 64], nh)
        start += 64
    assert torch.equal(out2, out[:192])
    # cached step == prefill for the target rows (prefix K/V as segment 0)
    out_c = torch.full_like(tq[P:], float("nan"))
    bd.sdpa_fwd(qr[P:], [kr[:P].clone(), kr[P:]], [tv[:P].clone(), tv[P:]], out_c, nh)
    assert bd.device_status() == 0
    G.check(G.host(out_c), G.host(out[P:]), max_abs=1e-2, what="cached vs prefill")


def test_sd15_self_and_cross_attention_core(bd, oracle):
    """SD1.5 at 512 px: 4096 tokens, 8 heads x 40; cross-attention to 77 keys."""
    nh, hd, L, Lc = 8, 40, 4096, 77
    D = nh * hd
    q = synth.activations((L, D), 1001)
    k = synth.activations((L, D), 1002)
    v = synth.activations((L, D), 1003)
    rows = G.boundary_rows(L, tile=32, extra=12)
    out = G.sdpa(bd, q, k, v, nh)
    G.check(out[rows], oracle.sdpa(q, k, v, nh, rows=rows), what="sd15 self")
    kc = synth.activations((Lc, D), 1004)
    vc = synth.activations((Lc, D), 1005)
    outc = G.sdpa(bd, q, kc, vc, nh)
    G.check(outc[rows], oracle.sdpa(q, kc, vc, nh, rows=rows), what="sd15 cross")
    # FP16 storage (the reference's SD1.5 GPU dtype)
    q16, k16, v16 = (synth.round_fp16(x[:256]) for x in (q, k, v))
    o16 = G.sdpa(bd, q16, k16, v16, nh, dtype=torch.float16)
    G.check(o16, oracle.sdpa(q16, k16, v16, nh), what="sd15 fp16")


def test_flux_2048_batch2_shape_properties(bd, oracle):
    """Flux.1 at 2048 px on one GPU (B = 2, 16896 tokens, 24 x 128): too large for
    the oracle in full, so check a few rows of the second batch item plus
    determinism."""
    nh, hd, L, B = 24, 128, 16896, 2
    D = nh * hd
    gen = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn(B, L, D, device="cuda", dtype=torch.bfloat16, generator=gen)
               for _ in range(3))
    out = torch.empty_like(q)
    bd.sdpa_fwd(q, k, v, out, nh)
    out2 = torch.empty_like(q)
    bd.sdpa_fwd(q, k, v, out2, nh)
    assert bd.device_status() == 0
    assert torch.equal(out, out2)
    rows = np.asarray([0, 127, 128, 255, 256, 8191, 16895], np.int32)
    ref = oracle.sdpa(G.host(q[1]), G.host(k[1]), G.host(v[1]), nh, rows=rows)
    G.check(G.host(out[1])[rows], ref, what="flux2048 batch item 1")


def test_sana_and_pixart_cross_attention_head_dims(bd, oracle):
    """Head dims 72 (Sana 0.6B / PixArt cross-attention, src/dit/sana.cpp:599-631,
    src/dit/pixart.cpp:359-365) and 112 (Sana 1.6B) run on the tensor-core kernel
    with the head zero-padded by the TMA unit; 300 caption keys with a key mask."""
    for nh, hd in ((16, 72), (20, 112)):
        Lq, Lk = 1024, 300
        q = synth.activations((Lq, nh * hd), 9000 + hd)
        k = synth.activations((Lk, nh * hd), 9001 + hd)
        v = synth.activations((Lk, nh * hd), 9002 + hd)
        km = np.ones(Lk, np.float32); km[200:] = 0.0
        rows = G.boundary_rows(Lq, extra=8)
        out = G.sdpa(bd, q, k, v, nh, key_mask=km)
        G.check(out[rows], oracle.sdpa(q, k, v, nh, key_mask=km, rows=rows), what=f"hd={hd} masked cross-attn")


@pytest.mark.parametrize("nq,nkv,hd", [(8, 2, 128), (6, 3, 64), (4, 1, 80), (4, 2, 160)])
def test_grouped_query_heads_without_widening(bd, oracle, nq, nkv, hd):
    """Krea 2 attention (dit::gqa_attention_masked, src/dit/common.cpp:331-377):
    K/V carry nkv heads and the kernel maps query head h to K/V head h // group;
    the oracle widens K/V as the reference does.  Key mask as in the text-fusion
    call, ragged length, both kernels (hd 160 takes the general one)."""
    L = 333
    q = synth.activations((L, nq * hd), 9700 + hd)
    k = synth.activations((L, nkv * hd), 9701 + hd)
    v = synth.activations((L, nkv * hd), 9702 + hd)
    km = np.ones(L, np.float32); km[::5] = 0.0
    for mask in (None, km):
        out = G.sdpa(bd, q, k, v, nq, num_kv_heads=nkv, key_mask=None if mask is None else mask.copy())
        ref = oracle.gqa_attention_masked(q, k, v, None, None, hd, nq, nkv, key_mask=mask)
        G.check(out, ref, what=f"gqa {nq}/{nkv} x{hd} mask={mask is not None}")
    # equal head counts are plain multi-head attention
    out = G.sdpa(bd, q, synth.activations((L, nq * hd), 9703), synth.activations((L, nq * hd), 9704), nq, num_kv_heads=nq)
    ref = oracle.sdpa(q, synth.activations((L, nq * hd), 9703), synth.activations((L, nq * hd), 9704), nq)
    G.check(out, ref, what="gqa with equal head counts")


def test_grouped_query_heads_refusals(bd):
    q = torch.zeros(64, 8 * 64, device="cuda", dtype=torch.bfloat16)
    kv = torch.zeros(64, 3 * 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match="num_kv_heads must divide num_heads"):
        bd.sdpa_fwd(q, kv, kv, torch.empty_like(q), 8, num_kv_heads=3)
    kv2 = torch.zeros(64, 2 * 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match="smaller than num_kv_heads"):
        bd.sdpa_fwd(q, kv2, kv2, torch.empty_like(q), 8, num_kv_heads=4)


@pytest.mark.parametrize("nh,hd,axes", [(2, 128, (16, 56, 56)), (3, 64, (8, 28, 28)), (2, 40, (8, 16, 16))])
def test_query_norm_and_rope_inside_the_kernel(bd, oracle, nh, hd, axes):
    """The Q half of the RMSNorm + RoPE pre-pass done by the attention kernel on
    its own query tiles (headnorm + rope_apply of Q, src/dit/flux.cpp:462-469,
    src/dit/common.cpp:192): text and image query segments with their own gains
    (norm_added_q / norm_q), table rows offset per segment, ragged image length;
    K is normalised and rotated beforehand as in the pre-pass.  Checked against
    the oracle and against the pre-pass path."""
    txt, hp, wp = 77, 18, 17
    img = hp * wp
    D = nh * hd
    q = synth.activations((txt + img, D), 9900 + hd)
    k = synth.activations((txt + img, D), 9901 + hd)
    v = synth.activations((txt + img, D), 9902 + hd)
    g_txt, g_img = synth.gains(hd, 9903, "f32"), synth.gains(hd, 9904, "f32")
    cos, sin = oracle.flux_rope_tables(txt, hp, wp, hd, axes)
    # oracle: norm + rope of Q per segment, K likewise (one gain is enough for K here)
    def nr(x, g, r0):
        return oracle.rope_apply(oracle.rms_norm_heads(x, nh, hd, g), nh, hd, cos[r0:], sin[r0:])
    qr = np.concatenate([nr(q[:txt], g_txt, 0), nr(q[txt:], g_img, txt)])
    kr = synth.round_bf16(np.concatenate([nr(k[:txt], g_txt, 0), nr(k[txt:], g_img, txt)]))
    ref = oracle.sdpa(synth.round_bf16(qr), kr, v, nh)
    tq, tk, tv = G.dev(q), G.dev(kr), G.dev(v)
    tcos, tsin = G.dev(cos, torch.float32), G.dev(sin, torch.float32)
    out = torch.full_like(tq, float("nan"))
    bd.sdpa_fwd([tq[:txt], tq[txt:]], tk, tv, [out[:txt], out[txt:]], nh,
                q_norm=dict(gain=[G.dev(g_txt, torch.float32), G.dev(g_img, torch.float32)], cos=tcos, sin=tsin))
    assert bd.device_status() == 0
    G.check(G.host(out), ref, what=f"fused query norm+rope hd={hd}")
    # the pre-pass path on the same inputs
    tqr = torch.empty_like(tq)
    bd.rmsnorm_rope([dict(x=tq[:txt], out=tqr[:txt], gain=G.dev(g_txt, torch.float32), cos=tcos, sin=tsin, rope_row0=0),
                     dict(x=tq[txt:], out=tqr[txt:], gain=G.dev(g_img, torch.float32), cos=tcos, sin=tsin, rope_row0=txt)],
                    nh, hd)
    out2 = torch.full_like(tq, float("nan"))
    bd.sdpa_fwd(tqr, tk, tv, out2, nh)
    assert (out.float() - out2.float()).abs().max().item() < 4e-3
    # RoPE only (no gains), one segment, rows offset into the table
    out3 = torch.full_like(tq[txt:], float("nan"))
    bd.sdpa_fwd(tq[txt:], tk, tv, out3, nh, q_norm=dict(gain=None, cos=tcos, sin=tsin, rope_row0=txt))
    ref3 = oracle.sdpa(synth.round_bf16(oracle.rope_apply(q[txt:], nh, hd, cos[txt:], sin[txt:])), kr, v, nh)
    G.check(G.host(out3), ref3, what=f"fused query rope only hd={hd}")


def test_fused_allgather_on_one_gpu_with_local_stand_in_peers(bd, oracle):
    """The head-sharded call (bdattn_sdpa_fwd_allgather) on ONE GPU: the "peers" are
    three more buffers on the same device, so the peer-store epilogue runs where only
    one GPU is at hand.  Every copy must equal the plain call bit for bit; shapes
    cover more CTAs than SMs, two query segments with a ragged tail, batch 2, and the
    masked and scaled instantiations."""
    nh, hd, B, txt, img = 4, 128, 2, 200, 5000          # (1 + 20) query CTAs x 4 heads x 2 = 168 items > 148 SMs
    L, D = txt + img, nh * hd
    gen = torch.Generator(device="cuda").manual_seed(4242)
    q, k, v = (torch.randn(B, L, D, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(3))
    seg = lambda t: [t[:, :txt], t[:, txt:]]
    ref = torch.empty_like(q)
    bd.sdpa_fwd(seg(q), seg(k), seg(v), seg(ref), nh)
    copies = [torch.full_like(q, float("nan")) for _ in range(4)]
    ptrs = lambda row0: [c[:, row0:].data_ptr() for c in copies[1:]]
    bd.sdpa_fwd(seg(q), seg(k), seg(v), seg(copies[0]), nh, peer_out_ptrs=[ptrs(0), ptrs(txt)])
    assert bd.device_status() == 0
    for i, c in enumerate(copies):
        assert torch.equal(c, ref), f"copy {i} differs from the plain call"
    # against the oracle on a few rows of batch item 1
    rows = G.boundary_rows(L, extra=4)[:10]
    o = oracle.sdpa(G.host(q[1]), G.host(k[1]), G.host(v[1]), nh, rows=rows)
    G.check(G.host(copies[2][1])[rows], o, what="gathered copy vs oracle")
    # causal + key mask, one segment, head dim 64
    nh2, hd2, L2 = 3, 64, 700
    q2, k2, v2 = (torch.randn(L2, nh2 * hd2, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(3))
    km = torch.ones(L2, device="cuda")
    km[100:140] = 0
    ref2 = torch.empty_like(q2)
    bd.sdpa_fwd(q2, k2, v2, ref2, nh2, mask_mode=bd.MASK_CAUSAL, key_mask=km)
    c2 = [torch.full_like(q2, float("nan")) for _ in range(3)]
    bd.sdpa_fwd(q2, k2, v2, c2[0], nh2, mask_mode=bd.MASK_CAUSAL, key_mask=km,
                peer_out_ptrs=[[c.data_ptr() for c in c2[1:]]])
    # per-key scale vectors together with the peer stores
    ks = torch.ones(L2, device="cuda")
    ks[:128] = 0.5
    ref3 = torch.empty_like(q2)
    bd.sdpa_fwd(q2, k2, v2, ref3, nh2, key_scale=ks, val_scale=ks)
    c3 = [torch.full_like(q2, float("nan")) for _ in range(3)]
    bd.sdpa_fwd(q2, k2, v2, c3[0], nh2, key_scale=ks, val_scale=ks,
                peer_out_ptrs=[[c.data_ptr() for c in c3[1:]]])
    assert bd.device_status() == 0
    for c in c2:
        assert torch.equal(c, ref2)
    for c in c3:
        assert torch.equal(c, ref3)


# --------------------------------------------------------------- edge cases
@pytest.mark.parametrize("hd", [128, 64, 40, 72, 112, 160])
@pytest.mark.parametrize("L", [1, 63, 64, 65, 127, 129, 257])
def test_ragged_lengths(bd, oracle, L, hd):
    nh = 2
    D = nh * hd
    Lq = L if L % 8 == 0 or True else L
    q = synth.activations((Lq, D), 4000 + L)
    k = synth.activations((L + 3, D), 4100 + L)
    v = synth.activations((L + 3, D), 4200 + L)
    G.check(G.sdpa(bd, q, k, v, nh), oracle.sdpa(q, k, v, nh), what=f"L={L} hd={hd}")
    G.check(G.sdpa(bd, q, k, v, nh, mask_mode=bd.MASK_CAUSAL),
            oracle.sdpa(q, k, v, nh, mask_mode=1), what=f"causal L={L} hd={hd}")


def test_odd_text_length_segments(bd, oracle):
    nh, hd, txt, img = 2, 128, 77, 300
    D = nh * hd
    q, k, v = (synth.activations((txt + img, D), 4300 + i) for i in range(3))
    out = G.sdpa(bd, [q[:txt], q[txt:]], [k[:txt], k[txt:]], [v[:txt], v[txt:]], nh)
    G.check(out, oracle.sdpa(q, k, v, nh), what="odd text length")


@pytest.mark.parametrize("hd", [128, 40])
def test_all_keys_masked_gives_zeros(bd, hd):
    nh, L = 2, 150
    q, k, v = (synth.activations((L, nh * hd), 4400 + i) for i in range(3))
    out = G.sdpa(bd, q, k, v, nh, key_mask=np.zeros(L, np.float32))
    assert np.all(out == 0.0)


@pytest.mark.parametrize("hd", [128, 64, 40])
def test_causal_with_more_queries_than_keys(bd, oracle, hd):
    """q_offset < 0: the first queries see no key at all and must give 0 (every
    exponential of such a row must be exactly zero, whichever way it is computed)."""
    nh = 2
    q = synth.activations((300, nh * hd), 4501)
    k = synth.activations((200, nh * hd), 4502)
    v = synth.activations((200, nh * hd), 4503)
    out = G.sdpa(bd, q, k, v, nh, mask_mode=bd.MASK_CAUSAL)
    ref = oracle.sdpa(q, k, v, nh, mask_mode=1)
    assert np.all(ref[:100] == 0.0)
    assert np.all(out[:100] == 0.0)
    G.check(out, ref, what="negative q_offset")


def test_large_logits_do_not_overflow(bd, oracle):
    nh, hd, L = 2, 128, 384
    q = synth.round_bf16(6.0 * synth.normal((L, nh * hd), 4601))
    k = synth.round_bf16(6.0 * synth.normal((L, nh * hd), 4602))
    v = synth.activations((L, nh * hd), 4603)
    G.check(G.sdpa(bd, q, k, v, nh), oracle.sdpa(q, k, v, nh), max_abs=4e-2, what="large logits")


# ------------------------------------------------------------- error surface
def test_argument_errors_carry_the_operator_prefix(bd):
    q = torch.zeros(16, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_sdpa_fwd: "):
        bd.sdpa_fwd(q, q, q, q, 3)                      # 256 / 3 is not a head dim
    with pytest.raises(bd.BdattnError, match=r"^bdattn_sdpa_fwd: "):
        bd.sdpa_fwd(q.float(), q.float(), q.float(), q.float(), 2)   # FP32 is refused
    with pytest.raises(bd.BdattnError, match=r"^bdattn_sdpa_fwd: .*aligned"):
        bd.sdpa_fwd(q[:, 1:129], q[:, :128], q[:, :128], q[:, :128].clone(), 1)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_sdpa_fwd: unknown mask_mode"):
        bd.sdpa_fwd(q, q, q, q.clone(), 2, mask_mode=7)
    # the multicast gather refuses an unaligned multicast address and head dims of the general kernel
    with pytest.raises(bd.BdattnError, match=r"^bdattn_sdpa_fwd_allgather_multicast: .*16-byte aligned"):
        bd.sdpa_fwd(q, q, q, q.clone(), 2, multicast_out_ptrs=[q.data_ptr() + 2])
    q192 = torch.zeros(16, 192, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_sdpa_fwd_allgather_multicast: .*head_dim <= 128"):
        bd.sdpa_fwd(q192, q192, q192, q192.clone(), 1, multicast_out_ptrs=[q192.data_ptr()])
