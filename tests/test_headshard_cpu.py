"""Host-side logic of the head-sharded path, with two gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from brodiffusion_b200 import headshard


def test_head_range_partitions():
    for nh, world in ((24, 1), (24, 2), (24, 4), (24, 8), (70, 2)):
        got = [headshard.head_range(nh, world, r) for r in range(world)]
        assert got[0][0] == 0 and got[-1][1] == nh
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
        assert len({b - a for a, b in got}) == 1
    with pytest.raises(ValueError):
        headshard.head_range(24, 5, 0)
    with pytest.raises(ValueError):
        headshard.head_range(24, 4, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        sys.path.insert(0, root)
        from oracle import oracle as O
        nh, hd, B, L = 4, 8, 2, 24
        D = nh * hd
        rng = np.random.default_rng(7)          # same data on every rank
        q, k, v = (rng.standard_normal((B, L, D)).astype(np.float32) for _ in range(3))
        wo = rng.standard_normal((D, D)).astype(np.float32) * 0.1
        h0, h1 = headshard.head_range(nh, world, rank)
        cols = slice(h0 * hd, h1 * hd)
        staging = torch.zeros(headshard.staging_shape(world, B, L, nh, hd))
        for b in range(B):                       # this rank's heads only
            o = O.sdpa(q[b][:, cols], k[b][:, cols], v[b][:, cols], h1 - h0)
            staging[rank, b] = torch.from_numpy(o)
        headshard.all_gather_heads(staging)
        full = np.stack([O.sdpa(q[b], k[b], v[b], nh) for b in range(B)])
        err_layout = float(np.abs(headshard.unstage(staging).numpy() - full).max())
        y = headshard.project_staged(staging, torch.from_numpy(wo)).numpy()
        err_proj = float(np.abs(y - full @ wo.T).max())
        ret[rank] = (err_layout, err_proj)
    finally:
        dist.destroy_process_group()


def test_two_rank_all_gather_matches_unsharded_oracle():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            err_layout, err_proj = ret[r]
            assert err_layout < 1e-6, f"rank {r}: gathered layout differs by {err_layout}"
            assert err_proj < 1e-4, f"rank {r}: staged projection differs by {err_proj}"
