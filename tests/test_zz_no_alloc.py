"""bdattn_qkvo_fwd_static: the SD1.5 attention block with its scratch in a
fixed array inside the library, for callers that may not allocate device
memory (a plugin whose host owns all of HBM, a loop where cudaMalloc is banned).

The entry point runs the same kernels as bdattn_qkvo_fwd, so its output is
compared with that entry point's on the same inputs, within the tolerance the
other GPU tests use; two different calls are made back to back to show that
what one call leaves in the shared array does not leak into the next.  The file
name sorts last so that a run that stops at the first failure has already run
every other test; it also passes on its own in a fresh process.
"""
import numpy as np
import pytest
import torch

import gpu_util as G
import synth

pytestmark = pytest.mark.gpu


def _both(bd, x, ctx, wq, wk, wv, wo, bo, nh, cached=None):
    """Run the caller-scratch entry point and the static one on the same data."""
    d = lambda a: G.dev(a) if a is not None else None
    tx, tctx = d(x), d(ctx)
    hd = wq.shape[0] // nh
    Lk = cached[0].shape[0] if cached is not None else (ctx.shape[0] if ctx is not None else x.shape[0])
    ws = torch.empty(bd.qkvo_workspace_bytes(x.shape[0], Lk, nh, hd), device="cuda", dtype=torch.uint8)
    kc, vc = (d(cached[0]), d(cached[1])) if cached is not None else (None, None)
    outs = []
    for workspace in (ws, None):     # None -> bdattn_qkvo_fwd_static
        out = torch.full((x.shape[0], wo.shape[0]), float("nan"), device="cuda", dtype=torch.bfloat16)
        bd.qkvo_fwd(tx, tctx, d(wq), d(wk), d(wv), d(wo), d(bo), nh, out, workspace,
                    k_cached=kc, v_cached=vc)
        assert bd.device_status() == 0
        outs.append(G.host(out))
    return outs


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row(bd, oracle):
    # call 1: the largest SD1.5 case, self-attention over 4096 tokens, 8 x 40
    L, C, nh = 4096, 320, 8
    x = synth.activations((L, C), 8001)
    wq, wk, wv, wo = (synth.weights((C, C), 8002 + i) for i in range(4))
    bo = synth.weights((C,), 8010)
    assert bd.qkvo_workspace_bytes(L, L, nh, C // nh) <= bd.qkvo_static_capacity()
    ref, got = _both(bd, x, None, wq, wk, wv, wo, bo, nh)
    G.check(got, ref, what="static vs caller scratch, self-attention")
    rows = G.boundary_rows(L, extra=4)
    q = oracle.linear(x[rows], wq)
    o = oracle.sdpa(q, oracle.linear(x, wk), oracle.linear(x, wv), nh)
    G.check(got[rows], oracle.linear(o, wo, bo), what="static scratch vs oracle")

    # call 2, straight after: a smaller, different problem (cross-attention with
    # cached K/V of 77 rows) that reuses the front of the same array
    Lq, Lc = 1024, 77
    x2 = synth.activations((Lq, C), 8101)
    kc = synth.activations((Lc, C), 8102)
    vc = synth.activations((Lc, C), 8103)
    ref2, got2 = _both(bd, x2, None, wq, None, None, wo, bo, nh, cached=(kc, vc))
    G.check(got2, ref2, what="static vs caller scratch, cached cross-attention")

    # and call 1 again gives what it gave the first time
    _, again = _both(bd, x, None, wq, wk, wv, wo, bo, nh)
    G.check(again, got, what="repeat of call 1")


def test_second_call_leaves_free_device_memory_unchanged(bd):
    """What the name promises: once the first call on the device has looked up the
    built-in array, a call changes the amount of free device memory by nothing.
    Inputs, outputs and torch's caching allocator are set up before the
    measurement; cudaMemGetInfo is read around the call itself."""
    L, C, nh = 1024, 320, 8
    x = torch.randn(L, C, device="cuda").bfloat16()
    ws = [torch.randn(C, C, device="cuda").bfloat16() * 0.05 for _ in range(4)]
    out = torch.empty(L, C, device="cuda", dtype=torch.bfloat16)
    bd.qkvo_fwd(x, None, ws[0], ws[1], ws[2], ws[3], None, nh, out, None)      # first call: set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        bd.qkvo_fwd(x, None, ws[0], ws[1], ws[2], ws[3], None, nh, out, None)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert bd.device_status() == 0
    assert free1 == free0, f"free device memory changed by {free0 - free1} bytes across calls"


def test_shapes_beyond_the_built_in_scratch_are_refused(bd):
    L, C, nh = 16384, 320, 8
    assert bd.qkvo_workspace_bytes(L, L, nh, C // nh) > bd.qkvo_static_capacity()
    x = torch.zeros(L, C, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(C, C, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(bd.BdattnError, match=r"^bdattn_qkvo_fwd_static: this call needs \d+ bytes of "
                                             r"scratch but the built-in array holds \d+"):
        bd.qkvo_fwd(x, None, w, w, w, w, None, nh, torch.empty_like(x), None)
