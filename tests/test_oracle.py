"""The CPU oracle against the golden fixtures (PyTorch float64, written from
the reference formulas) and against the relational checks the reference's own
tests make on this path."""
import numpy as np
import pytest

from conftest import bf16_from_bits, compare

TOL = 2e-5  # float32 oracle vs float64 fixture


def test_flux_rope_tables_match_golden(oracle, golden):
    cos, sin = oracle.flux_rope_tables(3, 4, 4, 8, (2, 2, 4))
    assert np.abs(cos - golden["flux_cos"]).max() < 1e-6
    assert np.abs(sin - golden["flux_sin"]).max() < 1e-6


def test_flux_rope_tables_known_answers(oracle):
    # text rows are the identity rotation; image (i, j) -> (0, i, j)
    # (src/dit/common.cpp:160-173); axis 0 is always position 0.
    cos, sin = oracle.flux_rope_tables(512, 8, 8, 128, (16, 56, 56))
    assert cos.shape == (512 + 64, 64)
    assert np.all(cos[:512] == 1.0) and np.all(sin[:512] == 0.0)
    assert np.all(cos[:, :8] == 1.0) and np.all(sin[:, :8] == 0.0)
    r = 512 + 3 * 8 + 5  # i = 3, j = 5
    assert cos[r, 8] == pytest.approx(np.cos(3.0), abs=1e-6)       # row axis, p = 0
    assert sin[r, 8 + 28] == pytest.approx(np.sin(5.0), abs=1e-6)  # col axis, p = 0
    w = 10000.0 ** (-2.0 * 3 / 56)
    assert cos[r, 8 + 3] == pytest.approx(np.cos(3.0 * w), abs=1e-6)
    with pytest.raises(ValueError):
        oracle.flux_rope_tables(1, 2, 2, 8, (2, 2, 2))  # axes do not sum to head_dim


def test_qwen_rope_tables_match_golden(oracle, golden):
    prefix = [("text", 5), ("image", 2, 3), ("text", 4)]
    cos, sin = oracle.qwen_rope_tables(prefix, 4, 4, 64, (8, 28, 28))
    assert cos.shape == golden["qwen_cos"].shape
    assert np.abs(cos - golden["qwen_cos"]).max() < 1e-6
    assert np.abs(sin - golden["qwen_sin"]).max() < 1e-6


def test_rms_norm_and_rope_match_golden(oracle, golden):
    qn = oracle.rms_norm_heads(golden["flux_q"], 2, 8, golden["flux_gq"], 1e-6)
    assert np.abs(qn - golden["flux_qn"]).max() < TOL
    qr = oracle.rope_apply(qn, 2, 8, golden["flux_cos"], golden["flux_sin"])
    assert np.abs(qr - golden["flux_qr"]).max() < TOL


def test_rope_half_split_is_a_permutation_of_interleaved(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 2 * 8)).astype(np.float32)
    cos, sin = oracle.flux_rope_tables(1, 2, 2, 8, (2, 2, 4))
    perm = np.concatenate([np.arange(0, 8, 2), np.arange(1, 8, 2)])   # interleaved -> split
    xs = x.reshape(5, 2, 8)[:, :, perm].reshape(5, 16)
    a = oracle.rope_apply(x, 2, 8, cos, sin, 0).reshape(5, 2, 8)[:, :, perm].reshape(5, 16)
    b = oracle.rope_apply(xs, 2, 8, cos, sin, 1)
    assert np.abs(a - b).max() < 1e-6


def test_flux_joint_attention_matches_golden(oracle, golden):
    g = golden
    qn = oracle.rms_norm_heads(g["flux_q"], 2, 8, g["flux_gq"])
    kn = oracle.rms_norm_heads(g["flux_k"], 2, 8, g["flux_gk"])
    out, avg = oracle.joint_attention(qn, kn, g["flux_v"], g["flux_cos"], g["flux_sin"], 8, 2,
                                      want_avg=True)
    assert np.abs(out - g["flux_out"]).max() < TOL
    assert np.abs(avg - g["flux_avg"]).max() < TOL
    # traced map rows are non-negative and sum to one
    # (tests/test_flux_blocks.cpp:268-281, tests/test_unet.cpp:487-500)
    assert avg.min() >= 0.0 and np.abs(avg.sum(1) - 1.0).max() < 1e-5
    # image->text logit bias (src/dit/common.cpp:259-281)
    outb = oracle.joint_attention(qn, kn, g["flux_v"], g["flux_cos"], g["flux_sin"], 8, 2,
                                  bias=g["flux_bias"], bias_row0=3)
    assert np.abs(outb - g["flux_out_biased"]).max() < TOL


def test_fast_variant_agrees_with_precise(oracle, golden):
    g = golden
    q, k, v = (bf16_from_bits(g[f"hd128_{n}_bf16"]) for n in "qkv")
    a = oracle.sdpa(q, k, v, 2, precise=True)
    b = oracle.sdpa(q, k, v, 2, precise=False)
    assert np.abs(a - b).max() < 1e-5


def test_masks_match_golden(oracle, golden):
    g = golden
    q, k, v = (bf16_from_bits(g[f"hd128_{n}_bf16"]) for n in "qkv")
    o = oracle.sdpa(q, k, v, 2, mask_mode=1)
    assert np.abs(o - g["hd128_out_causal"]).max() < TOL
    o = oracle.sdpa(q, k, v, 2, key_mask=g["hd128_keymask"])
    assert np.abs(o - g["hd128_out_keymask"]).max() < TOL
    # all keys masked -> zeros (inv = denom > 0 ? 1/denom : 0, common.cpp:293)
    o = oracle.sdpa(q, k, v, 2, key_mask=np.zeros(k.shape[0], np.float32))
    assert np.all(o == 0.0)
    # row subset selects the same rows
    rows = np.array([0, 7, 39], np.int32)
    sub = oracle.sdpa(q, k, v, 2, mask_mode=1, rows=rows)
    full = oracle.sdpa(q, k, v, 2, mask_mode=1)
    assert np.array_equal(sub, full[rows])


def _qwen_inputs(oracle, g):
    qr = oracle.rope_apply(oracle.rms_norm_heads(g["qwen_q"], 2, 64, g["qwen_gq"]), 2, 64,
                           g["qwen_cos"], g["qwen_sin"])
    kr = oracle.rope_apply(oracle.rms_norm_heads(g["qwen_k"], 2, 64, g["qwen_gk"]), 2, 64,
                           g["qwen_cos"], g["qwen_sin"])
    return qr, kr, g["qwen_v"]


def test_qwen_block_causal_matches_golden(oracle, golden):
    g = golden
    qr, kr, v = _qwen_inputs(oracle, g)
    assert np.abs(kr - g["qwen_kr"]).max() < TOL
    segs = [("text", 5), ("image", 6), ("text", 4), ("image", 16)]
    seg_id, is_img = oracle.block_causal_tables(segs)
    out = oracle.sdpa(qr, kr, v, 2, mask_mode=2, seg_id=seg_id, seg_is_image=is_img)
    assert np.abs(out - g["qwen_out"]).max() < TOL


def test_qwen_prefill_as_segment_calls_equals_block_causal(oracle, golden):
    """The reference runs the block-causal prefill as one attention call per
    prefix segment plus one for the target
    (src/dit/qwenimage21_forward.cpp:650-676); that composition must equal the
    mask rule, and the cached step (prefix K/V + fresh target rows) must equal
    the target rows of the full prefill (tests/test_qwenimage21_dit.cpp:117-128)."""
    g = golden
    qr, kr, v = _qwen_inputs(oracle, g)
    segs = [("text", 5), ("image", 6), ("text", 4)]
    out = np.zeros_like(qr)
    start = 0
    for kind, n in segs:
        end = start + n
        out[start:end] = oracle.sdpa(qr[start:end], kr[:end], v[:end], 2,
                                     mask_mode=1 if kind == "text" else 0)
        start = end
    out[start:] = oracle.sdpa(qr[start:], kr, v, 2)
    assert np.abs(out - g["qwen_out"]).max() < TOL
    # cached step: queries = target rows, keys = [cached prefix ; fresh target]
    cached = oracle.sdpa(qr[start:], np.concatenate([kr[:start], kr[start:]]),
                         np.concatenate([v[:start], v[start:]]), 2)
    assert np.array_equal(cached, out[start:])


def test_four_text_blocks_of_64_equal_one_causal_run(oracle):
    """The Qwen-Image configuration words the prefix as causal blocks of 64: four text segments of
    64 are the same visibility rule as one text run of 256."""
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((256, 2 * 16)).astype(np.float32) for _ in range(3))
    one = oracle.sdpa(q, k, v, 2, mask_mode=1)
    four = np.concatenate([oracle.sdpa(q[s:s + 64], k[:s + 64], v[:s + 64], 2, mask_mode=1)
                           for s in range(0, 256, 64)])
    assert np.array_equal(one, four)


def test_sd15_attention_matches_golden(oracle, golden):
    g = golden
    o = oracle.qkvo_attention(g["sd_x"], None, g["sd_wq"], g["sd_wk"], g["sd_wv"], g["sd_wo"],
                              g["sd_bo"], 4)
    assert np.abs(o - g["sd_self_out"]).max() < 5e-5
    o = oracle.qkvo_attention(g["sd_x"], g["sd_ctx"], g["sd_wq"], g["sd_wk2"], g["sd_wv2"],
                              g["sd_wo"], g["sd_bo"], 4)
    assert np.abs(o - g["sd_cross_out"]).max() < 5e-5


def test_sana_linear_attention_matches_golden(oracle, golden):
    g = golden
    out, sz = oracle.sana_linear_attn(g["sana_q"], g["sana_k"], g["sana_v"], 2, 32, want_sz=True)
    err, cos = compare(out, g["sana_out"])
    assert err < 1e-4 and cos > 0.999999
    assert np.abs(sz - g["sana_sz"]).max() < 1e-4
    # inject seam: adding w * own state scales numerator and denominator alike
    out2 = oracle.sana_linear_attn(g["sana_q"], g["sana_k"], g["sana_v"], 2, 32, sz_in=sz, w_in=0.5)
    assert np.abs(out2 - out).max() < 1e-4


def test_geglu_matches_golden(oracle, golden):
    g = golden
    y = oracle.linear_geglu(g["geglu_x"], g["geglu_w"], g["geglu_b"])
    assert np.abs(y - g["geglu_y"]).max() < 1e-5


def test_oracle_matches_torch_sdpa(oracle):
    """Independent second opinion: PyTorch's own FP32 CPU attention."""
    import torch
    rng = np.random.default_rng(11)
    L, nh, hd = 96, 3, 40
    q, k, v = (rng.standard_normal((L, nh * hd)).astype(np.float32) for _ in range(3))
    tq, tk, tv = (torch.from_numpy(a).view(L, nh, hd).transpose(0, 1) for a in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(tq, tk, tv)
    ref = ref.transpose(0, 1).reshape(L, -1).numpy()
    assert np.abs(oracle.sdpa(q, k, v, nh) - ref).max() < 2e-6


def test_gqa_matches_torch_grouped_attention(oracle):
    """dit::gqa_attention_masked restated (K/V heads widened, then plain
    attention) against PyTorch's FP32 grouped-query attention."""
    import torch
    rng = np.random.default_rng(12)
    L, nq, nkv, hd = 70, 6, 2, 24
    q = rng.standard_normal((L, nq * hd)).astype(np.float32)
    k, v = (rng.standard_normal((L, nkv * hd)).astype(np.float32) for _ in range(2))
    tq = torch.from_numpy(q).view(L, nq, hd).transpose(0, 1)
    tk, tv = (torch.from_numpy(a).view(L, nkv, hd).transpose(0, 1) for a in (k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(tq, tk, tv, enable_gqa=True)
    ref = ref.transpose(0, 1).reshape(L, -1).numpy()
    got = oracle.gqa_attention_masked(q, k, v, None, None, hd, nq, nkv)
    assert np.abs(got - ref).max() < 2e-6
    with pytest.raises(ValueError):
        oracle.gqa_attention_masked(q, k, v, None, None, hd, nq, 4)
