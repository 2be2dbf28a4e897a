"""Per-head RMSNorm + RoPE kernel against the oracle (C ABI, GPU)."""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu

# One BF16 rounding of values up to ~5: half an ulp at 4..8 is 2^-6.
TOL = 1.6e-2


def _run(bd, x, nh, hd, gain=None, cos=None, sin=None, row0=0, pair_mode=0, gain_f32=True,
         dtype=torch.bfloat16, inplace=False):
    tx = G.dev(x, dtype)
    out = tx if inplace else torch.full_like(tx, float("nan"))
    job = dict(x=tx, out=out, rope_row0=row0)
    if gain is not None:
        job["gain"] = G.dev(gain, torch.float32 if gain_f32 else dtype)
    if cos is not None:
        job["cos"], job["sin"] = G.dev(cos, torch.float32), G.dev(sin, torch.float32)
    bd.rmsnorm_rope([job], nh, hd, pair_mode=pair_mode)
    assert bd.device_status() == 0
    return G.host(out)


@pytest.mark.parametrize("hd,axes", [(128, (16, 56, 56)), (64, (8, 28, 28)), (8, (2, 2, 4))])
def test_norm_then_rope(bd, oracle, hd, axes):
    nh, txt, hp, wp = 3, 5, 6, 7
    L = txt + hp * wp
    x = synth.activations((L, nh * hd), 5000 + hd)
    g = synth.gains(hd, 5100 + hd)
    cos, sin = oracle.flux_rope_tables(txt, hp, wp, hd, axes)
    ref = oracle.rope_apply(oracle.rms_norm_heads(x, nh, hd, g), nh, hd, cos, sin)
    got = _run(bd, x, nh, hd, g, cos, sin)
    assert np.abs(got - ref).max() < TOL
    # gain at the tensor dtype (Flux) instead of FP32 (Qwen-Image)
    got = _run(bd, x, nh, hd, g, cos, sin, gain_f32=False)
    assert np.abs(got - ref).max() < TOL
    # in place
    got = _run(bd, x, nh, hd, g, cos, sin, inplace=True)
    assert np.abs(got - ref).max() < TOL


def test_norm_only_and_rope_only(bd, oracle):
    nh, hd, L = 2, 128, 40
    x = synth.activations((L, nh * hd), 5201)
    g = synth.gains(hd, 5202)
    cos, sin = oracle.flux_rope_tables(8, 4, 8, hd)
    assert np.abs(_run(bd, x, nh, hd, gain=g) - oracle.rms_norm_heads(x, nh, hd, g)).max() < TOL
    assert np.abs(_run(bd, x, nh, hd, cos=cos, sin=sin) -
                  oracle.rope_apply(x, nh, hd, cos, sin)).max() < TOL


def test_rope_row_offset_and_half_split(bd, oracle):
    """Qwen-Image cached step: target rows use table rows offset by the prefix
    length (src/dit/qwenimage21_forward.cpp:305-307)."""
    nh, hd = 2, 128
    cos, sin = oracle.qwen_rope_tables([("text", 9)], 4, 4, hd)
    x = synth.activations((16, nh * hd), 5301)
    ref = oracle.rope_apply(x, nh, hd, cos[9:], sin[9:])
    assert np.abs(_run(bd, x, nh, hd, cos=cos, sin=sin, row0=9) - ref).max() < TOL
    ref = oracle.rope_apply(x, nh, hd, cos[9:], sin[9:], pair_mode=1)
    assert np.abs(_run(bd, x, nh, hd, cos=cos, sin=sin, row0=9, pair_mode=1) - ref).max() < TOL


def test_four_jobs_in_one_launch_and_strided_rows(bd, oracle):
    nh, hd = 2, 64
    D = nh * hd
    xs = [synth.activations((r, D), 5400 + i) for i, r in enumerate((3, 50, 1, 17))]
    gs = [synth.gains(hd, 5410 + i) for i in range(4)]
    wide = [torch.zeros(x.shape[0], 3 * D, device="cuda", dtype=torch.bfloat16) for x in xs]
    jobs = []
    for x, g, w in zip(xs, gs, wide):
        w[:, D:2 * D] = G.dev(x)
        jobs.append(dict(x=w[:, D:2 * D], out=w[:, D:2 * D], gain=G.dev(g, torch.float32)))
    bd.rmsnorm_rope(jobs, nh, hd)
    assert bd.device_status() == 0
    for x, g, w in zip(xs, gs, wide):
        assert np.abs(G.host(w[:, D:2 * D]) - oracle.rms_norm_heads(x, nh, hd, g)).max() < TOL
        assert torch.count_nonzero(w[:, :D]) == 0 and torch.count_nonzero(w[:, 2 * D:]) == 0


def test_fp16_storage(bd, oracle):
    nh, hd, L = 2, 40, 33
    x = synth.activations((L, nh * hd), 5501, "fp16")
    g = synth.gains(hd, 5502, "f32")
    ref = oracle.rms_norm_heads(x, nh, hd, g)
    assert np.abs(_run(bd, x, nh, hd, gain=g, dtype=torch.float16) - ref).max() < 4e-3


def test_errors(bd):
    x = torch.zeros(4, 256, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(4, 64, device="cuda")
    with pytest.raises(bd.BdattnError, match=r"^bdattn_rmsnorm_rope: .*cos and sin"):
        bd.rmsnorm_rope([dict(x=x, out=x, cos=c)], 2, 128)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_rmsnorm_rope: n_jobs"):
        bd.rmsnorm_rope([dict(x=x, out=x)] * 5, 2, 128)
