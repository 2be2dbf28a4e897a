"""Writes ``ref_pin.npz``: outputs of brodiffusion's own ``src/dit/common.cpp``
(compiled unmodified as ``oracle/_ref/libref.so``) on small seeded inputs.

Run where the brodiffusion source tree is present:
    python tests/golden/make_ref_pin.py
The fixture lets ``tests/test_oracle_pin.py`` check the oracle restatement
against the reference's own arithmetic on hosts that do not have that tree.
Cases follow the reference's tiny-Flux test configuration
(tests/test_flux_blocks.cpp:480-507: 2 heads x 8, axes_dims_rope {2, 2, 4})
and one case at the Flux.1 head shape (head_dim 128, axes {16, 56, 56}).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import synth  # noqa: E402
from oracle import ref  # noqa: E402

CASES = {
    # name: (txt_len, hp, wp, heads, head_dim, axes, with_bias)
    "tiny": (5, 4, 3, 2, 8, (2, 2, 4), True),
    "tiny_nobias": (3, 2, 2, 2, 8, (2, 2, 4), False),
    "flux_head": (7, 5, 6, 2, 128, (16, 56, 56), True),
}


def inputs(name):
    txt, hp, wp, nh, hd, axes, with_bias = CASES[name]
    L, D = txt + hp * wp, nh * hd
    seed = 9000 + 10 * sorted(CASES).index(name)
    q, k, v = (synth.activations((L, D), seed + i) for i in range(3))
    bias = synth.activations((hp * wp, txt), seed + 5) if with_bias else None
    return q, k, v, bias


def main():
    ref.build()
    out = {}
    for name, (txt, hp, wp, nh, hd, axes, with_bias) in CASES.items():
        cos, sin = ref.flux_rope_tables(txt, hp, wp, hd, axes)
        q, k, v, bias = inputs(name)
        # identity tables: the attention core alone (rope_apply belongs to brotensor)
        L = txt + hp * wp
        one, zero = np.ones((L, hd // 2), np.float32), np.zeros((L, hd // 2), np.float32)
        o, avg = ref.joint_attention_traced(q, k, v, one, zero, hd, nh, txt, bias)
        out[f"{name}_cos"], out[f"{name}_sin"] = cos, sin
        out[f"{name}_out"], out[f"{name}_avg"] = o, avg
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_pin.npz"), **out)
    print("wrote ref_pin.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
