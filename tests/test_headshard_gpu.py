"""Head-sharded attention on 2 GPUs (config 5 layout, reduced size): the NCCL
all-gather path, the fused peer-store path and the fused multicast-store path
(when the group has an NVLink multicast address) against the unsharded kernel.
Needs two GPUs; skipped on a single-GPU box."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import brodiffusion_b200 as bd
        from brodiffusion_b200 import headshard
        nh, hd, B, txt, img = 8, 128, 2, 64, 448
        L, D = txt + img, nh * hd
        gen = torch.Generator(device=dev).manual_seed(77)      # same data on every rank
        q, k, v = (torch.randn(B, L, D, device=dev, dtype=torch.bfloat16, generator=gen) for _ in range(3))
        # unsharded result (all heads on this GPU)
        full = torch.empty_like(q)
        bd.sdpa_fwd([q[:, :txt], q[:, txt:]], [k[:, :txt], k[:, txt:]], [v[:, :txt], v[:, txt:]],
                    [full[:, :txt], full[:, txt:]], nh)
        h0, h1 = headshard.head_range(nh, world, rank)
        cols = slice(h0 * hd, h1 * hd)
        ql, kl, vl = q[:, :, cols], k[:, :, cols], v[:, :, cols]
        # (a) NCCL all-gather of head-major slabs
        staging = torch.zeros(headshard.staging_shape(world, B, L, nh, hd), device=dev, dtype=torch.bfloat16)
        out = staging[rank]
        bd.sdpa_fwd([ql[:, :txt], ql[:, txt:]], [kl[:, :txt], kl[:, txt:]], [vl[:, :txt], vl[:, txt:]],
                    [out[:, :txt], out[:, txt:]], h1 - h0)
        headshard.all_gather_heads(staging)
        ok_nccl = torch.equal(headshard.unstage(staging), full)
        # (b) fused: the epilogue stores into every rank's replica
        go = headshard.GatheredOutput(B, L, nh, hd, torch.bfloat16, dev)
        go.full.fill_(float("nan"))
        go.barrier()
        lo = go.local
        bd.sdpa_fwd([ql[:, :txt], ql[:, txt:]], [kl[:, :txt], kl[:, txt:]], [vl[:, :txt], vl[:, txt:]],
                    [lo[:, :txt], lo[:, txt:]], h1 - h0,
                    peer_out_ptrs=[go.peer_ptrs(0), go.peer_ptrs(txt)])
        go.barrier()
        ok_fused = torch.equal(go.full, full)
        # (c) fused through the switch: one multimem.st per vector reaches every replica
        have = torch.tensor([1 if go.multicast_ptr(0) else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(have, op=dist.ReduceOp.MIN)
        ok_mc = None
        if int(have.item()) == 1:
            go.full.fill_(float("nan"))
            go.barrier()
            bd.sdpa_fwd([ql[:, :txt], ql[:, txt:]], [kl[:, :txt], kl[:, txt:]], [vl[:, :txt], vl[:, txt:]],
                        [lo[:, :txt], lo[:, txt:]], h1 - h0,
                        multicast_out_ptrs=[go.multicast_ptr(0), go.multicast_ptr(txt)])
            go.barrier()
            ok_mc = bool(torch.equal(go.full, full))
        status = bd.device_status()
        ret[rank] = (bool(ok_nccl), bool(ok_fused), int(status), ok_mc)
    finally:
        dist.destroy_process_group()


def test_two_gpu_head_sharding_matches_unsharded():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        for r in range(world):
            ok_nccl, ok_fused, status, ok_mc = ret[r]
            assert status == 0
            assert ok_nccl, f"rank {r}: NCCL all-gather result differs from the unsharded kernel"
            assert ok_fused, f"rank {r}: fused all-gather result differs from the unsharded kernel"
            assert ok_mc is not False, f"rank {r}: multicast all-gather result differs from the unsharded kernel"
