"""Prefix KV cache operations of the Qwen-Image path on the device
(QwenImage21PrefixCache::scale_kv / ::blend_from,
src/dit/qwenimage21_hooks.cpp:79-124) and their effect on the cached
attention step."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16).cpu().numpy()


@pytest.mark.parametrize("shape", [(256, 3072), (77, 123), (1, 5)])
def test_scale_and_blend_are_bit_exact(bd, oracle, shape):
    k0 = synth.activations(shape, 9800)
    k1 = synth.activations(shape, 9801)
    tk = G.dev(k0)
    bd.axpby_inplace(tk, None, 0.37)                        # scale_kv
    ref = oracle.prefix_cache_scale(k0, 0.37, synth.round_bf16)
    assert np.array_equal(_bits(tk), _bits(G.dev(ref)))
    bd.axpby_inplace(tk, G.dev(k1), 1.0 - 0.25, 0.25)        # blend_from, alpha = 0.25
    ref = oracle.prefix_cache_blend(ref, k1, 0.25, synth.round_bf16)
    assert bd.device_status() == 0
    assert np.array_equal(_bits(tk), _bits(G.dev(ref)))


def test_fp16_and_identity_cases(bd, oracle):
    y0 = synth.round_fp16(synth.normal((40, 72), 9810))
    x = synth.round_fp16(synth.normal((40, 72), 9811))
    ty = G.dev(y0, torch.float16)
    bd.axpby_inplace(ty, None, 1.0)                          # scale 1: untouched (hooks.cpp:91,94)
    assert np.array_equal(G.host(ty), y0)
    bd.axpby_inplace(ty, G.dev(x, torch.float16), 0.5, 0.5)
    ref = oracle.prefix_cache_blend(y0, x, 0.5, synth.round_fp16)
    assert np.array_equal(G.host(ty), ref)
    with pytest.raises(bd.BdattnError, match="x is null"):
        bd.axpby_inplace(ty, None, 1.0, 0.5)


def test_cached_step_with_scaled_cache_equals_scale_hooks(bd, oracle):
    """Scaling the cache in place and attending equals attending with the
    key_scale / val_scale hooks of the un-scaled cache up to the one extra
    rounding of the stored cache (src/dit/qwenimage21_forward.cpp:606-645)."""
    nh, hd, P, T = 4, 128, 256, 512
    D = nh * hd
    q = synth.activations((T, D), 9820)
    kc, vc = synth.activations((P, D), 9821), synth.activations((P, D), 9822)
    kf, vf = synth.activations((T, D), 9823), synth.activations((T, D), 9824)
    tkc, tvc = G.dev(kc), G.dev(vc)
    bd.axpby_inplace(tkc, None, 1.5)
    bd.axpby_inplace(tvc, None, 0.5)
    out = torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
    bd.sdpa_fwd(G.dev(q), [tkc, G.dev(kf)], [tvc, G.dev(vf)], out, nh)
    assert bd.device_status() == 0
    ks = oracle.prefix_cache_scale(kc, 1.5, synth.round_bf16)
    vs = oracle.prefix_cache_scale(vc, 0.5, synth.round_bf16)
    ref = oracle.sdpa(q, np.concatenate([ks, kf]), np.concatenate([vs, vf]), nh)
    G.check(G.host(out), ref, what="cached step over a scaled prefix cache")
    # the hooks on the un-scaled cache: the kernel scales the prefix rows of its K / V
    # tiles in shared memory and rounds them to BF16 like scale_inplace does, so the
    # two ways agree bit for bit
    ksv, vsv = np.ones(P + T, np.float32), np.ones(P + T, np.float32)
    ksv[:P], vsv[:P] = 1.5, 0.5
    out_h = torch.empty_like(out)
    bd.sdpa_fwd(G.dev(q), [G.dev(kc), G.dev(kf)], [G.dev(vc), G.dev(vf)], out_h, nh,
                key_scale=G.dev(ksv, torch.float32), val_scale=G.dev(vsv, torch.float32))
    assert bd.device_status() == 0
    assert torch.equal(out_h, out)
    # and with a key mask on top (the scale and mask hooks together)
    km = np.ones(P + T, np.float32)
    km[P + 100:P + 130] = 0.0
    out_m = torch.empty_like(out)
    bd.sdpa_fwd(G.dev(q), [G.dev(kc), G.dev(kf)], [G.dev(vc), G.dev(vf)], out_m, nh,
                key_scale=G.dev(ksv, torch.float32), val_scale=G.dev(vsv, torch.float32),
                key_mask=G.dev(km, torch.float32))
    assert bd.device_status() == 0
    ref_m = oracle.sdpa(q, np.concatenate([ks, kf]), np.concatenate([vs, vf]), nh, key_mask=km)
    G.check(G.host(out_m), ref_m, what="scaled prefix cache with a key mask")
