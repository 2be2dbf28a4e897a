"""Helpers for the GPU parity tests: move numpy data through the C ABI."""
import numpy as np
import torch

import synth

MAX_ABS = 2e-2     # parity bound of the path: BF16 GPU vs FP32 CPU oracle
MIN_COS = 0.9999


def dev(x, dtype=torch.bfloat16):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(dtype)


def host(t):
    return t.float().cpu().numpy()


def sdpa(bd, q, k, v, nh, dtype=torch.bfloat16, **kw):
    """q, k, v: numpy arrays or lists of numpy arrays (row segments)."""
    def up(x):
        return [dev(a, dtype) for a in x] if isinstance(x, (list, tuple)) else dev(x, dtype)
    tq, tk, tv = up(q), up(k), up(v)
    if isinstance(tq, list):
        out = [torch.full_like(a, float("nan")) for a in tq]
    else:
        out = torch.full_like(tq, float("nan"))
    for name in ("key_mask", "key_scale", "val_scale"):
        if kw.get(name) is not None:
            kw[name] = dev(kw[name], torch.float32)
    bd.sdpa_fwd(tq, tk, tv, out, nh, **kw)
    assert bd.device_status() == 0
    if isinstance(out, list):
        return np.concatenate([host(o) for o in out])
    return host(out)


def boundary_rows(L, tile=128, extra=24, seed=0):
    """Query rows to check on a large case: every tile edge neighbourhood is
    too many, so take the first/last rows, rows around a few tile edges and a
    seeded random sample."""
    rows = {0, 1, L - 1, L - 2}
    for e in (tile, 2 * tile, 4 * tile, (L // tile) * tile):
        for d in (-1, 0, 1):
            if 0 <= e + d < L:
                rows.add(e + d)
    u = synth.uniform01(extra, 9000 + seed)
    rows.update(int(x * L) for x in u)
    return np.asarray(sorted(r for r in rows if 0 <= r < L), np.int32)


def check(got, ref, max_abs=MAX_ABS, min_cos=MIN_COS, what=""):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - ref).max()
    cos = (got * ref).sum() / (np.sqrt((got * got).sum() * (ref * ref).sum()) + 1e-300)
    assert err <= max_abs, f"{what}: max-abs error {err:.5f} > {max_abs}"
    assert cos >= min_cos, f"{what}: cosine {cos:.6f} < {min_cos}"
    return err, cos
