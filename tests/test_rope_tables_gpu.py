"""Device-built RoPE tables against the oracle / golden tables."""
import numpy as np
import pytest

import gpu_util as G

pytestmark = pytest.mark.gpu


def test_flux_tables(bd, oracle, golden):
    cos, sin = bd.rope_tables_flux(3, 4, 4, 8, (2, 2, 4))
    assert bd.device_status() == 0
    assert np.abs(G.host(cos) - golden["flux_cos"]).max() < 1e-6
    assert np.abs(G.host(sin) - golden["flux_sin"]).max() < 1e-6
    for txt, hp, wp in ((512, 64, 64), (512, 128, 128), (0, 5, 7), (9, 0, 0)):
        cos, sin = bd.rope_tables_flux(txt, hp, wp, 128)
        rc, rs = oracle.flux_rope_tables(txt, hp, wp, 128)
        assert np.abs(G.host(cos) - rc).max() < 2e-6
        assert np.abs(G.host(sin) - rs).max() < 2e-6


def test_qwen_tables(bd, oracle, golden):
    prefix = [("text", 5), ("image", 2, 3), ("text", 4)]
    cos, sin = bd.rope_tables_qwen(prefix, 4, 4, 64, (8, 28, 28))
    assert bd.device_status() == 0
    assert np.abs(G.host(cos) - golden["qwen_cos"]).max() < 1e-6
    assert np.abs(G.host(sin) - golden["qwen_sin"]).max() < 1e-6
    for prefix in ([("text", 256)], [("image", 8, 8)] * 4, []):
        cos, sin = bd.rope_tables_qwen(prefix, 64, 64, 128)
        rc, rs = oracle.qwen_rope_tables(prefix, 64, 64, 128)
        assert cos.shape == rc.shape
        # positions reach ~4400 on the frame axis: FP32 rounding of the angle
        assert np.abs(G.host(cos) - rc).max() < 2e-6
        assert np.abs(G.host(sin) - rs).max() < 2e-6


def test_errors_keep_the_reference_messages(bd):
    with pytest.raises(bd.BdattnError, match="build_axial_rope_tables: axes_dims_rope must sum to head_dim"):
        bd.rope_tables_flux(1, 2, 2, 8, (2, 2, 2))
    with pytest.raises(bd.BdattnError, match="build_axial_rope_tables: head_dim must be even"):
        bd.rope_tables_flux(1, 2, 2, 7, (2, 2, 3))
