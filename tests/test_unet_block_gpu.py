"""SD1.5 transformer-block operators on the GPU: fused QKVO attention (self,
cross, cached K/V), the K/V cache projection, fused FF1 + GEGLU and the two
residual adds, each against the golden fixtures and the oracle.  Bounds for
the fused ops are the reference's own (tests/test_fused_parity.cpp:168-239):
0.01 * max|ref| + 0.008 for GEGLU, 0.005 * max|ref| + 0.003 for the adds."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu


def _qkvo(bd, x, ctx, wq, wk, wv, wo, bo, nh, dtype=torch.bfloat16, cached=None, **kw):
    d = lambda a: G.dev(a, dtype) if a is not None else None
    tx, tctx = d(x), d(ctx)
    out = torch.full((x.shape[0], wo.shape[0]), float("nan"), device="cuda", dtype=dtype)
    hd = wq.shape[0] // nh
    Lk = cached[0].shape[0] if cached is not None else (ctx.shape[0] if ctx is not None else x.shape[0])
    ws = torch.empty(bd.qkvo_workspace_bytes(x.shape[0], Lk, nh, hd), device="cuda", dtype=torch.uint8)
    kc, vc = (d(cached[0]), d(cached[1])) if cached is not None else (None, None)
    bd.qkvo_fwd(tx, tctx, d(wq), d(wk), d(wv), d(wo), d(bo), nh, out, ws, k_cached=kc, v_cached=vc, **kw)
    assert bd.device_status() == 0
    return G.host(out)


def test_golden_tiny_self_and_cross(bd, golden):
    g = golden
    r = synth.round_bf16
    args = [r(g[k]) for k in ("sd_x", "sd_ctx", "sd_wq", "sd_wk", "sd_wv", "sd_wo", "sd_wk2", "sd_wv2", "sd_bo")]
    x, ctx, wq, wk, wv, wo, wk2, wv2, bo = args
    out = _qkvo(bd, x, None, wq, wk, wv, wo, bo, 4)
    G.check(out, g["sd_self_out"], max_abs=6e-2, min_cos=0.999, what="tiny self (bf16 weights)")
    out = _qkvo(bd, x, ctx, wq, wk2, wv2, wo, bo, 4)
    G.check(out, g["sd_cross_out"], max_abs=6e-2, min_cos=0.999, what="tiny cross (bf16 weights)")


@pytest.mark.parametrize("L,C,nh", [(4096, 320, 8), (1024, 640, 8), (256, 1280, 8), (64, 1280, 8)])
def test_sd15_self_attention_levels(bd, oracle, L, C, nh):
    """SD1.5 at 512 px and the deeper U-Net levels (src/unet.cpp:450): head dims 40,
    80 (padded to the tensor-core kernel) and 160 (general kernel)."""
    x = synth.activations((L, C), 7000 + L)
    wq, wk, wv, wo = (synth.weights((C, C), 7001 + L + i) for i in range(4))
    bo = synth.weights((C,), 7010 + L)
    rows = np.unique(np.concatenate([G.boundary_rows(L, extra=8), np.arange(min(L, 16))]))
    out = _qkvo(bd, x, None, wq, wk, wv, wo, bo, nh)
    # oracle on the sampled rows: project everything, attend sampled rows
    q = oracle.linear(x[rows], wq)
    k, v = oracle.linear(x, wk), oracle.linear(x, wv)
    o = oracle.sdpa(q, k, v, nh)
    ref = oracle.linear(o, wo, bo)
    G.check(out[rows], ref, what=f"self L={L} C={C}")


def test_sd15_cross_attention_uncached_cached_and_project_kv(bd, oracle):
    L, C, nh, Lc, Cc = 4096, 320, 8, 77, 768
    x = synth.activations((L, C), 7101)
    ctx = synth.activations((Lc, Cc), 7102)
    wq, wo = synth.weights((C, C), 7103), synth.weights((C, C), 7104)
    wk, wv = synth.weights((C, Cc), 7105), synth.weights((C, Cc), 7106)
    bo = synth.weights((C,), 7107)
    rows = G.boundary_rows(L, extra=8)
    ref = oracle.qkvo_attention(x[rows], ctx, wq, wk, wv, wo, bo, nh)
    out = _qkvo(bd, x, ctx, wq, wk, wv, wo, bo, nh)
    G.check(out[rows], ref, what="cross uncached")
    # K/V cache primed once per prompt (src/unet.cpp:458-495), then reused
    kc = torch.empty(Lc, C, device="cuda", dtype=torch.bfloat16)
    vc = torch.empty_like(kc)
    bd.project_kv(G.dev(ctx), G.dev(wk), G.dev(wv), kc, vc)
    assert bd.device_status() == 0
    G.check(G.host(kc), oracle.linear(ctx, wk), what="project_kv K")
    G.check(G.host(vc), oracle.linear(ctx, wv), what="project_kv V")
    out_c = _qkvo(bd, x, None, wq, None, None, wo, bo, nh, cached=(G.host(kc), G.host(vc)))
    G.check(out_c[rows], ref, what="cross cached")
    G.check(out_c, out, max_abs=1e-2, what="cached vs uncached")


def test_fp16_self_attention(bd, oracle):
    """The reference runs SD1.5 in FP16 on the GPU."""
    L, C, nh = 512, 320, 8
    x = synth.activations((L, C), 7201, "fp16")
    wq, wk, wv, wo = (synth.weights((C, C), 7202 + i, "fp16") for i in range(4))
    bo = synth.weights((C,), 7210, "fp16")
    out = _qkvo(bd, x, None, wq, wk, wv, wo, bo, nh, dtype=torch.float16)
    G.check(out, oracle.qkvo_attention(x, None, wq, wk, wv, wo, bo, nh), what="fp16 self")


def test_linear(bd, oracle):
    for (M, N, K) in ((4096, 320, 320), (77, 320, 768), (130, 72, 40), (1, 8, 8)):
        x = synth.activations((M, K), 7300 + M)
        w = synth.weights((N, K), 7301 + M)
        b = synth.weights((N,), 7302 + M)
        y = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        bd.linear_fwd(G.dev(x), G.dev(w), G.dev(b), y)
        assert bd.device_status() == 0
        G.check(G.host(y), oracle.linear(x, w, b), what=f"linear {M}x{N}x{K}")


@pytest.mark.parametrize("B,Din,Dout", [(40, 64, 48), (128, 128, 96), (4096, 320, 1280), (2300, 200, 1152)])
def test_fused_linear_geglu(bd, oracle, golden, B, Din, Dout):
    """Reference shapes (tests/test_fused_parity.cpp:268-269) plus the SD1.5
    top-level FF1 (4096, 320) -> 1280 and a ragged case; the last two are large
    enough for the persistent wide-tile kernel (value + gate tile per MMA)."""
    if (B, Din, Dout) == (40, 64, 48):
        x, w, b = golden["geglu_x"], golden["geglu_w"], golden["geglu_b"]
        ref = golden["geglu_y"]
    else:
        x = synth.activations((B, Din), 7400 + B, "fp16")
        w = synth.round_fp16(synth.normal((2 * Dout, Din), 7401 + B, 0, 0.1))
        b = synth.round_fp16(synth.normal((2 * Dout,), 7402 + B, 0, 0.2))
        ref = oracle.linear_geglu(x, w, b)
    y = torch.full((B, Dout), float("nan"), device="cuda", dtype=torch.float16)
    bd.linear_geglu_fwd(G.dev(x, torch.float16), G.dev(w, torch.float16), G.dev(b, torch.float16), y)
    assert bd.device_status() == 0
    got = G.host(y)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 0.01 * np.abs(ref).max() + 0.008


@pytest.mark.parametrize("rows,cols", [(10, 37), (64, 64), (4096, 320)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_add_inplace_vec(bd, rows, cols, dtype):
    rnd = synth.round_fp16 if dtype == torch.float16 else synth.round_bf16
    y0 = rnd(synth.uniform01(rows * cols, 7500).astype(np.float32).reshape(rows, cols) * 2 - 1)
    x = rnd(synth.uniform01(rows * cols, 7501).astype(np.float32).reshape(rows, cols) * 2 - 1)
    ty = G.dev(y0, dtype)
    bd.add_inplace(ty, G.dev(x, dtype))
    assert bd.device_status() == 0
    ref = y0 + x
    assert np.abs(G.host(ty) - ref).max() <= 0.005 * np.abs(ref).max() + 0.003 + (0.004 if dtype == torch.bfloat16 else 0)


@pytest.mark.parametrize("rows,cols", [(13, 29), (48, 80)])
def test_add_inplace_row_bias(bd, rows, cols):
    y0 = synth.round_fp16(synth.uniform01(rows * cols, 7600).astype(np.float32).reshape(rows, cols) * 2 - 1)
    b = synth.round_fp16(synth.uniform01(cols, 7601).astype(np.float32) * 2 - 1)
    ty = G.dev(y0, torch.float16)
    bd.add_row_bias(ty, G.dev(b, torch.float16))
    assert bd.device_status() == 0
    ref = y0 + b[None, :]
    assert np.abs(G.host(ty) - ref).max() <= 0.005 * np.abs(ref).max() + 0.003


def test_errors(bd):
    x = torch.zeros(16, 320, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(320, 320, device="cuda", dtype=torch.bfloat16)
    small = torch.empty(16, device="cuda", dtype=torch.uint8)
    with pytest.raises(bd.BdattnError, match=r"^flash_attention_qkvo_forward: workspace of \d+ bytes needed"):
        bd.qkvo_fwd(x, None, w, w, w, w, None, 8, torch.empty_like(x), small)
    with pytest.raises(bd.BdattnError, match=r"^fused_linear_geglu: tensors must be FP16 or BF16"):
        xf = x.float()
        bd.linear_geglu_fwd(xf, xf, None, xf.clone())
    # an output whose rows are narrower than what one row receives would be overwritten
    y = torch.empty(16 * 320, device="cuda", dtype=torch.bfloat16).as_strided((16, 320), (160, 1))
    with pytest.raises(bd.BdattnError, match=r"^bdattn_linear_fwd: output row stride 160 is smaller than the 320 columns"):
        bd.linear_fwd(x, w, None, y)
    # a bad cached K/V is refused before anything is enqueued: the output stays as it was
    ws = torch.empty(bd.qkvo_workspace_bytes(16, 77, 8, 40), device="cuda", dtype=torch.uint8)
    kc = torch.zeros(77, 324, device="cuda", dtype=torch.bfloat16)[:, 4:]      # rows start 8 bytes off a 16-byte boundary
    out = torch.full((16, 320), 7.0, device="cuda", dtype=torch.bfloat16)
    ws.zero_()
    with pytest.raises(bd.BdattnError, match=r"^flash_attention_q_with_kv_cached_forward: cached K/V must be 16-byte aligned"):
        bd.qkvo_fwd(x + 1, None, w + 1, None, None, w, None, 8, out, ws, k_cached=kc, v_cached=kc)
    torch.cuda.synchronize()
    assert bool((ws == 0).all()) and bool((out == 7.0).all())
