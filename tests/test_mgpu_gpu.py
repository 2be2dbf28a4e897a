"""bdattn_mgpu_*: several GPUs driven from ONE process with one host thread per
GPU, through the C ABI.  Head-sharded attention stores into every GPU's own copy
of the output; the cross-GPU barrier's wait is bounded and reports a missing rank
through the status word instead of hanging.  Needs two GPUs; skipped on a
single-GPU box.  NVLS / multimem are not involved (plain peer stores)."""
import threading

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _run_threads(fn, n):
    errs = [None] * n

    def wrap(r):
        try:
            torch.cuda.set_device(r)
            fn(r)
        except Exception as e:          # surfaced in the main thread below
            errs[r] = e

    ts = [threading.Thread(target=wrap, args=(r,)) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for e in errs:
        if e is not None:
            raise e


def test_headsharded_attention_fills_every_replica(bd):
    _need_two()
    G = 2
    nh, hd, B, txt, img = 8, 128, 2, 64, 448
    L, D = txt + img, nh * hd
    gen = torch.Generator().manual_seed(91)
    hq, hk, hv = (torch.randn(B, L, D, generator=gen).bfloat16() for _ in range(3))
    mg = bd.MultiGpu(list(range(G)))
    assert mg.size() == G
    replicas = [torch.full((B, L, D), float("nan"), device=f"cuda:{g}", dtype=torch.bfloat16) for g in range(G)]
    full = [None] * G
    status = [None] * G

    def work(r):
        dev = torch.device("cuda", r)
        q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
        ref = torch.empty_like(q)
        bd.sdpa_fwd([q[:, :txt], q[:, txt:]], [k[:, :txt], k[:, txt:]], [v[:, :txt], v[:, txt:]],
                    [ref[:, :txt], ref[:, txt:]], nh)                      # unsharded, all heads
        full[r] = ref
        per = nh // G
        cols = slice(r * per * hd, (r + 1) * per * hd)
        ql, kl, vl = q[:, :, cols], k[:, :, cols], v[:, :, cols]
        mg.barrier(r)                       # the NaN fill of every replica is complete
        mg.sdpa_fwd_headsharded(r, [ql[:, :txt], ql[:, txt:]], [kl[:, :txt], kl[:, txt:]],
                                [vl[:, :txt], vl[:, txt:]], replicas, nh)
        mg.barrier(r)
        torch.cuda.synchronize(dev)
        status[r] = bd.device_status()

    _run_threads(work, G)
    for r in range(G):
        assert status[r] == 0
        assert torch.equal(replicas[r], full[r]), f"replica {r} differs from the unsharded kernel"
    mg.destroy()


def test_barrier_wait_runs_out_when_a_rank_does_not_arrive(bd):
    """Rank 1 leaves between steps (it simply makes no barrier call; nothing of its
    is in flight).  Rank 0's wait gives up after its short limit, the kernel returns
    normally with BDATTN_STATUS_WAIT_TIMEOUT set, and the GPU keeps working."""
    _need_two()
    mg = bd.MultiGpu([0, 1])
    seen = {}

    def work(r):
        dev = torch.device("cuda", r)
        mg.barrier(r, timeout_ms=500)       # step 1: both arrive
        torch.cuda.synchronize(dev)
        seen[("first", r)] = bd.device_status()
        if r == 0:
            mg.barrier(r, timeout_ms=300)   # step 2: rank 1 never comes
            torch.cuda.synchronize(dev)
            seen["second"] = bd.device_status()
            x = torch.ones(1024, device=dev)
            seen["alive"] = float((x * 2).sum().item())
            seen["after"] = bd.device_status()

    _run_threads(work, 2)
    assert seen[("first", 0)] == 0 and seen[("first", 1)] == 0
    assert seen["second"] & bd.STATUS_WAIT_TIMEOUT
    assert seen["alive"] == 2048.0 and seen["after"] == 0      # the word was cleared, the context is usable
    mg.destroy()


def test_argument_errors(bd):
    with pytest.raises(bd.BdattnError, match=r"^bdattn_mgpu_init: n_gpus must be in \[1, 8\]"):
        bd.MultiGpu([])
    with pytest.raises(bd.BdattnError, match=r"^bdattn_mgpu_init: device 0 is listed twice"):
        bd.MultiGpu([0, 0])
    mg = bd.MultiGpu([0])
    torch.cuda.set_device(0)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_mgpu_barrier: rank 3 is not in \[0, 1\)"):
        mg.barrier(3)
    mg.barrier(0)                    # a group of one passes at once
    torch.cuda.synchronize()
    assert bd.device_status() == 0
    mg.destroy()
