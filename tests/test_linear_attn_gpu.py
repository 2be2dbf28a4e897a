"""Sana ReLU linear attention on the GPU against the golden fixture and the
oracle (FP32 statement of src/dit/sana.cpp:470-520)."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu


def _run(bd, q, k, v, nh, sz_in=None, w_in=0.0, want_sz=False):
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    out = torch.full_like(tq, float("nan"))
    B = q.shape[0] if q.ndim == 3 else 1
    szo = torch.full((B, nh, 33, 32), float("nan"), device="cuda") if want_sz else None
    szi = G.dev(sz_in, torch.float32) if sz_in is not None else None
    bd.linear_attn_relu_fwd(tq, tk, tv, out, nh, 32, sz_in=szi, w_in=w_in, sz_out=szo)
    assert bd.device_status() == 0
    return (G.host(out), G.host(szo)) if want_sz else G.host(out)


def test_golden(bd, golden):
    g = golden
    out, sz = _run(bd, g["sana_q"], g["sana_k"], g["sana_v"], 2, want_sz=True)
    G.check(out, g["sana_out"], what="sana golden")
    assert np.abs(sz[0] - g["sana_sz"]).max() < 1e-3 * np.abs(g["sana_sz"]).max()


@pytest.mark.parametrize("N,B", [(1024, 2), (4096, 2), (1024, 1), (4096, 1), (16384, 1)])
def test_sana_1600m_shapes(bd, oracle, N, B):
    """Sana 1600M: 70 heads x 32, 1024 / 4096 tokens, batch 2 (CFG) and the
    reference's own per-branch batch of 1 (which runs as a cluster of 2); 16384
    tokens (4096 px) walks the ring a dozen times per CTA."""
    nh, hd = 70, 32
    D = nh * hd
    q = synth.activations((B, D, N), 6001 + N)
    k = synth.activations((B, D, N), 6002 + N)
    v = synth.activations((B, D, N), 6003 + N)
    wo = synth.weights((D, D), 6004)
    out = _run(bd, q, k, v, nh)
    for b in range(B):
        ref = oracle.sana_linear_attn(q[b], k[b], v[b], nh, hd)
        o = out[b]
        G.check(o, ref, what=f"sana N={N} b={b}")
        # after the (token-major) output projection: (N, D) @ Wo^T
        G.check(o.T[:256] @ wo.T, ref.T[:256] @ wo.T, what="sana after out-projection")


@pytest.mark.parametrize("N", [1024, 4096])
def test_sana_projections_feed_the_core_channel_major(bd, oracle, N):
    """The three Sana projections at their real shape, q = W (2240, 2240) . x_mod (N, 2240)^T
    -> (2240, N) channel-major, bias-free (src/dit/sana.cpp:441-443: matmul_abt with
    W as the row operand), straight into the ReLU linear-attention core
    (src/dit/sana.cpp:521-586)."""
    nh, hd = 70, 32
    D = nh * hd
    x_mod = synth.activations((N, D), 6400 + N)
    ws = [synth.weights((D, D), 6410 + i) for i in range(3)]
    tx = G.dev(x_mod)
    qkv = []
    for w in ws:
        y = torch.full((D, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        bd.linear_fwd(G.dev(w), tx, None, y)          # rows of W against rows of x_mod
        qkv.append(y)
    assert bd.device_status() == 0
    ref_qkv = [oracle.linear(w, x_mod) for w in ws]    # (D, N)
    for name, y, r in zip("qkv", qkv, ref_qkv):
        # reference bound for a 16-bit GEMM against FP32 (tests/test_fused_parity.cpp:66-90)
        err = np.abs(G.host(y) - r).max()
        assert err <= 0.01 * np.abs(r).max() + 0.004, f"{name} projection: {err}"
    out = torch.full((D, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    bd.linear_attn_relu_fwd(qkv[0], qkv[1], qkv[2], out, nh, hd)
    assert bd.device_status() == 0
    # oracle on the device's own (BF16-rounded) projections: isolates the core ...
    ref = oracle.sana_linear_attn(G.host(qkv[0]), G.host(qkv[1]), G.host(qkv[2]), nh, hd)
    G.check(G.host(out), ref, what=f"sana core on projected q/k/v, N={N}")
    # ... and end to end from x_mod with FP32 projections
    ref_e2e = oracle.sana_linear_attn(ref_qkv[0], ref_qkv[1], ref_qkv[2], nh, hd)
    G.check(G.host(out), ref_e2e, max_abs=3e-2, min_cos=0.999, what=f"sana projections + core, N={N}")


@pytest.mark.parametrize("N", [8, 64, 120, 136, 520])
def test_ragged_token_counts(bd, oracle, N):
    nh = 3
    q, k, v = (synth.activations((nh * 32, N), 6100 + N + i) for i in range(3))
    G.check(_run(bd, q, k, v, nh), oracle.sana_linear_attn(q, k, v, nh, 32), what=f"N={N}")


def test_capture_and_inject_state(bd, oracle):
    """(S, z) identity seam: capture, then inject with a weight
    (src/dit/sana.cpp:492-509,550-559)."""
    nh, N = 4, 256
    q, k, v = (synth.activations((nh * 32, N), 6200 + i) for i in range(3))
    k2, v2 = (synth.activations((nh * 32, N), 6210 + i) for i in range(2))
    _, sz = _run(bd, q, k2, v2, nh, want_sz=True)
    ref_sz = oracle.sana_linear_attn(q, k2, v2, nh, 32, want_sz=True)[1]
    assert np.abs(sz[0] - ref_sz).max() < 1e-3 * np.abs(ref_sz).max()
    out = _run(bd, q, k, v, nh, sz_in=ref_sz, w_in=0.3)
    ref = oracle.sana_linear_attn(q, k, v, nh, 32, sz_in=ref_sz, w_in=0.3)
    G.check(out, ref, what="inject")


def test_back_to_back_launches_see_each_others_results(bd, oracle):
    """The kernel is launched with programmatic stream serialisation: its set-up
    may overlap the tail of the kernel before it.  Launches that depend on one
    another (the second reads the first's output as its queries; the third
    overwrites the buffer the second read) must give what separately synchronised
    launches give, every time."""
    nh, N = 70, 1024
    D = nh * 32
    q, k, v = (synth.activations((2, D, N), 6400 + i) for i in range(3))
    tq, tk, tv = G.dev(q), G.dev(k), G.dev(v)
    o1, o2 = torch.empty_like(tq), torch.empty_like(tq)
    # separately synchronised
    bd.linear_attn_relu_fwd(tq, tk, tv, o1, nh, 32)
    torch.cuda.synchronize()
    bd.linear_attn_relu_fwd(o1, tk, tv, o2, nh, 32)
    torch.cuda.synchronize()
    want1, want2 = o1.clone(), o2.clone()
    bd.linear_attn_relu_fwd(tq, tv, tk, o1, nh, 32)
    torch.cuda.synchronize()
    want3 = o1.clone()
    for _ in range(20):
        o1.fill_(float("nan"))
        o2.fill_(float("nan"))
        bd.linear_attn_relu_fwd(tq, tk, tv, o1, nh, 32)
        bd.linear_attn_relu_fwd(o1, tk, tv, o2, nh, 32)     # reads o1
        bd.linear_attn_relu_fwd(tq, tv, tk, o1, nh, 32)     # overwrites o1
        torch.cuda.synchronize()
        assert torch.equal(o2, want2)
        assert torch.equal(o1, want3)
    assert bd.device_status() == 0
    ref = oracle.sana_linear_attn(q[0], k[0], v[0], nh, 32)
    G.check(G.host(want1)[0], ref, what="first launch")


def test_all_negative_keys_give_zero(bd):
    nh, N = 2, 128
    q = synth.activations((nh * 32, N), 6301)
    k = -np.abs(synth.activations((nh * 32, N), 6302))
    v = synth.activations((nh * 32, N), 6303)
    out = _run(bd, q, k, v, nh)
    assert np.all(out == 0.0)     # 0 / (0 + 1e-15)


def test_errors(bd):
    x = torch.zeros(64, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_linear_attn_relu_fwd: head_dim must be 32"):
        bd.linear_attn_relu_fwd(x, x, x, x.clone(), 1, 64)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_linear_attn_relu_fwd: dtype must be BF16"):
        h = x.half()
        bd.linear_attn_relu_fwd(h, h, h, h.clone(), 2, 32)
