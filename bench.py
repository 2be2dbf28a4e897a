#!/usr/bin/env python
"""Benchmark of the denoiser-attention hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl ours|reference]
                  [--workload flux1024|flux2048_headsharded|sana1024|sana4096|flux1024_qkv_proj|flux1024_out_proj]

One step = one pass of the hot path over one synthetic batch:
  flux1024              (1 GPU)  Flux.1 joint attention at 1024 px, double-stream
                        form: per-head QK RMSNorm + 3-axis RoPE (one launch, four
                        jobs) and the joint softmax attention of 512 text + 4096
                        image tokens, 24 heads x 128 (one launch).  With --q-norm
                        fused the attention kernel normalises and rotates its own
                        query tiles and the pre-pass handles K only.
  flux2048_headsharded  (N GPUs) Flux.1 joint attention at 2048 px, batch 2,
                        512 + 16384 tokens; heads split over the ranks, all-gather
                        of the per-head outputs.  Default for N > 1.
  sana1024 / sana4096   (1 GPU)  Sana ReLU linear attention, batch 2 (GB/s).
  flux1024_qkv_proj / flux1024_out_proj  (1 GPU)  the projections either side of
                        the flux1024 attention call (projection TFLOP/s).
The metric is attention TFLOP/s with the reference's own FLOP convention
(4 * Lq * Lk * heads * head_dim, tools/bench_krea2_kernels.cpp:188-192).

Timing: W warm-up steps, then the K-step region (barrier + synchronize on both
sides, CUDA events on the launching stream, max over ranks) is measured R
times; ``ms_per_step`` is the median region and the minimum and maximum are
printed beside it.  SM clocks and throttle reasons are sampled across all R
regions.

The default one-GPU line also carries, measured in the same run after the
timed regions: ``also`` (the other configurations of the path: Sana linear
attention, the Qwen-Image cached step with and without the prefix scale
vectors, the SD1.5 self-attention block, the Flux projections) and
``library_baseline`` (torch SDPA and flash_attn on the same tensors).  A line
for N > 1 carries ``gather_check`` (rank 0 recomputes heads another rank owns
and compares them bit for bit with its gathered copy) and
``one_gpu_same_workload`` (rank 0 alone on the whole call, for a like-for-like
scaling figure).

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement
of the reference path (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

NH, HD = 24, 128
D = NH * HD
WORKLOADS = {
    # name: (batch, text rows, latent rows, latent cols)
    "flux1024": (1, 512, 64, 64),
    "flux2048_headsharded": (2, 512, 128, 128),
}
# Sana 1600M ReLU linear attention: name -> (batch, heads, tokens); 1 GPU, HBM-bound.
SANA_WORKLOADS = {"sana1024": (2, 70, 1024), "sana4096": (2, 70, 4096)}
PROJ_WORKLOADS = {"flux1024_qkv_proj": 3, "flux1024_out_proj": 1}
# dram__bytes_read.sum + dram__bytes_write.sum of one sdpa_tc05_kernel launch
# on the flux1024 workload, from one ncu capture of that launch.
NCU_TRAFFIC_BYTES = {"flux1024": 84.99e6 + 6.07e6}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def sustained_peak_tf():
    """cuBLAS BF16 rate of a seconds-long loop under the power cap (the figure for
    a kernel timed inside a long step), or the fallback for it."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return 1400.0


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only)."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._period = period_s
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self._period)

    def start(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_min_mhz": s[0] if s else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s),
                "sampled": "across the timed regions"}


def attention_flops(batch, L):
    return 4.0 * batch * L * L * D


def step_text(q_fused, world):
    s = ("rmsnorm+rope of K -> joint softmax attention (rmsnorm+rope of Q inside)" if q_fused
         else "rmsnorm+rope (Q,K) -> joint softmax attention")
    return s + (" -> all-gather of head outputs" if world > 1 else "")


def workload_config(args, world):
    """The ``config`` object of the line: what is computed, identical for the GPU
    arm and the host arm so that their lines describe the same job."""
    batch, txt, hp, wp = WORKLOADS[args.workload]
    L = txt + hp * wp
    return {"workload": args.workload, "batch": batch, "tokens": L, "text_tokens": txt, "heads": NH,
            "head_dim": HD, "heads_per_gpu": NH // world,
            "step": step_text(args.q_norm == "fused", world),
            "gather": "none" if world == 1 else
                      ("fused into the attention epilogue (stores to the switch's multicast address, or "
                       "to every peer) + symmetric-memory barrier"
                       if args.gather.startswith("fused") else "nccl all-gather"),
            "l2": "GPU arm: steps rotate over input sets that together exceed the 126 MB L2; "
                  "host arm: inputs are read from host memory"}


# ----------------------------------------------------------------- reference
def run_reference(args, rank, world):
    """CPU restatement of the reference path on the host cores (all threads)."""
    if rank != 0:
        return
    import numpy as np
    import synth
    from oracle import oracle as O
    O.build()
    batch, txt, hp, wp = WORKLOADS[args.workload]
    L = txt + hp * wp
    cores = O.hardware_threads()
    q = synth.activations((L, D), 11)
    k = synth.activations((L, D), 12)
    v = synth.activations((L, D), 13)
    # size one step to a bounded sample: aim for ~120 s in total
    probe_rows = np.arange(0, L, L // 16, dtype=np.int32)[:16]
    t0 = time.perf_counter()
    O.sdpa(q, k, v, NH, rows=probe_rows, precise=False)
    per_row = (time.perf_counter() - t0) / len(probe_rows)
    n_steps = args.steps + args.warmup
    rows_n = int(max(16, min(L, (120.0 / n_steps) / per_row)))
    rows = np.linspace(0, L - 1, rows_n).astype(np.int32)
    for _ in range(args.warmup):
        O.sdpa(q, k, v, NH, rows=rows, precise=False)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.sdpa(q, k, v, NH, rows=rows, precise=False)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 4.0 * rows_n * L * D / dt / 1e12
    sample = (f"{rows_n} of {L} query rows per step (all {NH} heads, all {L} keys), attention "
              f"core in FP32, batch item 0 of {batch}")
    line = {
        "impl": "reference", "metric": "attention TFLOP/s", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3,                                       # one measured sample step
        "full_call_ms_extrapolated": batch * L / rows_n * dt * 1e3,   # rows are independent
        "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args, max(1, args.gpus)),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------ timing helpers
def graph_ms(step, steps, reps=5, sampler=None):
    """Median per-step device time of ``steps`` calls replayed from a CUDA graph
    (host launch gaps do not enter the device time of microsecond kernels)."""
    import torch
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(steps):
                step(i)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    out = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / steps)
    if sampler is not None:
        t_end = time.perf_counter() + 0.2
        while time.perf_counter() < t_end:        # keep the GPU busy while the clock sampler collects
            graph.replay()
        torch.cuda.synchronize()
        sampler.stop()
    return statistics.median(out)


def measure_sana(bd, B, nh, N, steps=20, sampler=None):
    """Sana linear attention: (ms, algorithmic GB/s).  Algorithmic bytes =
    q, k, v read + out written = 4 * tokens * heads*32 * 2 bytes per batch item."""
    import torch
    Dm = nh * 32
    byt = 4.0 * B * Dm * N * 2
    n_sets = max(2, int(300e6 / byt) + 1)
    gen = torch.Generator(device="cuda").manual_seed(4321)
    sets = [tuple(torch.randn(B, Dm, N, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(3))
            for _ in range(n_sets)]
    outs = [torch.empty(B, Dm, N, device="cuda", dtype=torch.bfloat16) for _ in range(n_sets)]

    def step(i):
        q, k, v = sets[i % n_sets]
        bd.linear_attn_relu_fwd(q, k, v, outs[i % n_sets], nh, 32)

    ms = graph_ms(step, steps, sampler=sampler)
    return ms, byt / (ms * 1e-3) / 1e9, n_sets, byt


def measure_copy_same_bytes(B, nh, N, steps=20):
    """Context for the Sana figures, not a product path: a plain device-to-device copy
    (the library's copy kernel) that moves as many bytes as the linear attention does
    (2 tensors' worth read, 2 written), timed the same way (CUDA-graph replay of
    ``steps`` launches, buffers rotating over more than the L2).  Returns ms per launch."""
    import torch
    half = 2 * B * nh * 32 * N                 # elements read = elements written
    n_sets = max(2, int(300e6 / (4.0 * half)) + 1)
    src = [torch.empty(half, device="cuda", dtype=torch.bfloat16).normal_() for _ in range(n_sets)]
    dst = [torch.empty(half, device="cuda", dtype=torch.bfloat16) for _ in range(n_sets)]

    def step(i):
        dst[i % n_sets].copy_(src[i % n_sets])

    return graph_ms(step, steps)


def measure_proj(bd, n_proj, steps=20, sampler=None):
    """Projections around the Flux 1024 px attention call (4608 tokens, 3072 ->
    3072, BF16): n_proj = 3 is one bdattn_qkv_norm_rope_fwd call, 1 is one
    bdattn_linear_fwd call.  Returns (ms, TFLOP/s)."""
    import torch
    L, Dm, nh, hd = 4608, 3072, 24, 128
    gen = torch.Generator(device="cuda").manual_seed(9876)
    n_sets = 6                                   # 6 x 28 MB of activations > 126 MB L2
    xs = [torch.randn(L, Dm, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(n_sets)]
    W = [torch.randn(Dm, Dm, device="cuda", dtype=torch.bfloat16, generator=gen) * 0.02 for _ in range(n_proj)]
    outs = [torch.empty(L, Dm, device="cuda", dtype=torch.bfloat16) for _ in range(n_proj)]
    gain = torch.ones(hd, device="cuda", dtype=torch.bfloat16)
    cos, sin = bd.rope_tables_flux(512, 64, 64, hd)

    def step(i):
        x = xs[i % n_sets]
        if n_proj == 3:
            bd.qkv_norm_rope_fwd(x, W[0], W[1], W[2], outs[0], outs[1], outs[2], nh, hd, gain_q=gain, gain_k=gain,
                                 cos=cos, sin=sin)
        else:
            bd.linear_fwd(x, W[0], None, outs[0])

    ms = graph_ms(step, steps, sampler=sampler)
    return ms, n_proj * 2.0 * L * Dm * Dm / (ms * 1e-3) / 1e12


def measure_qwen_cached(bd, scaled, steps=10):
    """Qwen-Image cached step: 4096 fresh query rows against a 256-row prefix K/V
    cache (segment 0) plus the 4096 fresh rows, 24 x 128; ``scaled`` adds the
    prefix K and V attenuation vectors.  Returns (ms, TFLOP/s)."""
    import torch
    P, T = 256, 4096
    gen = torch.Generator(device="cuda").manual_seed(2468)
    n_sets = 3                                   # 3 x (q + 2 x (P + T) rows) x 6 KB > 126 MB L2
    sets = [(torch.randn(T, D, device="cuda", dtype=torch.bfloat16, generator=gen),
             torch.randn(P + T, D, device="cuda", dtype=torch.bfloat16, generator=gen),
             torch.randn(P + T, D, device="cuda", dtype=torch.bfloat16, generator=gen)) for _ in range(n_sets)]
    out = torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
    kw = {}
    if scaled:
        ks = torch.ones(P + T, device="cuda")
        vs = torch.ones(P + T, device="cuda")
        ks[:P], vs[:P] = 0.5, 0.25
        kw = dict(key_scale=ks, val_scale=vs)

    def step(i):
        q, k, v = sets[i % n_sets]
        bd.sdpa_fwd(q, [k[:P], k[P:]], [v[:P], v[P:]], out, NH, **kw)

    ms = graph_ms(step, steps)
    return ms, 4.0 * T * (P + T) * D / (ms * 1e-3) / 1e12


def measure_sd15_block(bd, steps=20):
    """SD1.5 self-attention block at 512 px (one CFG branch): x (4096, 320), 8 heads x
    40, Q/K/V projections + attention + output projection in one bdattn_qkvo_fwd
    call.  Returns (ms, TFLOP/s over core + projection FLOP)."""
    import torch
    L, C, nh = 4096, 320, 8
    gen = torch.Generator(device="cuda").manual_seed(1357)
    n_sets = 56                                  # 56 x 2.6 MB activations > 126 MB L2
    xs = [torch.randn(L, C, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(n_sets)]
    ws = [torch.randn(C, C, device="cuda", dtype=torch.bfloat16, generator=gen) * 0.05 for _ in range(4)]
    bo = torch.zeros(C, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(L, C, device="cuda", dtype=torch.bfloat16)
    wsp = torch.empty(bd.qkvo_workspace_bytes(L, L, nh, C // nh), device="cuda", dtype=torch.uint8)

    def step(i):
        bd.qkvo_fwd(xs[i % n_sets], None, ws[0], ws[1], ws[2], ws[3], bo, nh, out, wsp)

    ms = graph_ms(step, steps)
    flop = 4.0 * L * L * C + 4 * 2.0 * L * C * C
    return ms, flop / (ms * 1e-3) / 1e12


def other_configurations(bd):
    """The ``also`` block: the remaining configurations of the path, each timed
    for a few milliseconds in this same process."""
    peak_tf, peak_gbs, kind = measured_peaks()
    also = {"peaks": f"{kind}: {peak_tf} TFLOP/s BF16 burst, {peak_gbs} GB/s copy",
            "timing": "CUDA-graph replay, median of 5, inputs rotate over sets larger than L2"}

    def tensor(name, fn, what):
        try:
            ms, tf = fn()
            also[name] = {"ms": ms, "achieved": tf, "unit": "TFLOP/s", "frac": tf / peak_tf, "what": what}
        except Exception as e:          # a configuration that fails is reported, not hidden
            also[name] = {"error": f"{type(e).__name__}: {e}"}

    for name, (B, nh, N) in SANA_WORKLOADS.items():
        try:
            ms, gbs, _, _ = measure_sana(bd, B, nh, N)
            copy_ms = measure_copy_same_bytes(B, nh, N)
            also[name] = {"ms": ms, "achieved": gbs, "unit": "GB/s", "frac": gbs / peak_gbs,
                          "what": f"Sana ReLU linear attention, batch {B}, {nh} x 32, {N} tokens",
                          "copy_same_bytes_ms": copy_ms,
                          "copy_same_bytes": "library device-to-device copy of as many bytes, timed the same way "
                                             "(context: what a single streaming pass reaches at this size)"}
        except Exception as e:
            also[name] = {"error": f"{type(e).__name__}: {e}"}
    tensor("qwen_cached", lambda: measure_qwen_cached(bd, False),
           "Qwen-Image cached step, 4096 queries x (256 cached + 4096) keys, 24 x 128")
    tensor("qwen_cached_scaled", lambda: measure_qwen_cached(bd, True),
           "same with the prefix K and V scale vectors")
    tensor("sd15_self_block", lambda: measure_sd15_block(bd),
           "SD1.5 self-attention block 4096 x 320, 8 x 40: projections + attention + out-projection")
    tensor("flux1024_qkv_proj", lambda: measure_proj(bd, 3),
           "Q/K/V projections 4608 x 3072 -> 3 x 3072 with RMSNorm + RoPE in the epilogue")
    tensor("flux1024_out_proj", lambda: measure_proj(bd, 1), "output projection 4608 x 3072 x 3072")
    return also


def library_baselines(sets, batch, L, nh_l):
    """torch SDPA and flash_attn on the tensors of the timed workload (library
    kernels on the same box; context, not part of the product path)."""
    import torch
    res = {"what": "attention core only on the workload's tensors, median of 10, CUDA events"}
    flops = 4.0 * batch * L * L * nh_l * HD

    def timed(fn):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        ts = []
        for i in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(i)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    try:
        import torch.nn.functional as F
        views = [tuple(t.view(batch, L, nh_l, HD).transpose(1, 2) for t in s) for s in sets]
        ms = timed(lambda i: F.scaled_dot_product_attention(*views[i % len(views)]))
        res["torch_sdpa"] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12}
    except Exception as e:
        res["torch_sdpa"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    try:
        from flash_attn import flash_attn_func
        views = [tuple(t.view(batch, L, nh_l, HD) for t in s) for s in sets]
        ms = timed(lambda i: flash_attn_func(*views[i % len(views)]))
        res["flash_attn"] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12}
    except Exception as e:
        res["flash_attn"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    return res


# ---------------------------------------------------------------------- ours
def bind_host_to_gpu(local_rank):
    """Keeps this process (and with it the pinned staging buffers it allocates from here
    on) on the CPU cores next to its GPU, as NVML reports them, so that the uploads and
    downloads of the end-to-end figure do not cross sockets.  Reads NVML only; a host that
    refuses the affinity call, or an image without NVML, leaves things as they were.
    Returns a word for the JSON line."""
    try:
        import pynvml
        import torch
        pr = torch.cuda.get_device_properties(local_rank)
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByPciBusId(
            f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0".encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        near &= os.sched_getaffinity(0)
        if not near:
            return "unchanged (no usable cores reported next to the GPU)"
        os.sched_setaffinity(0, near)
        return f"{len(near)} cores next to the GPU"
    except Exception as e:
        return f"unchanged ({type(e).__name__})"


def run_ours(args, rank, world, local_rank):
    import numpy as np
    import torch
    import synth
    import brodiffusion_b200 as bd
    from brodiffusion_b200 import headshard

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    host_binding = bind_host_to_gpu(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    batch, txt, hp, wp = WORKLOADS[args.workload]
    L = txt + hp * wp
    h0, h1 = headshard.head_range(NH, world, rank)
    nh_l = h1 - h0
    d_l = nh_l * HD
    flops = attention_flops(batch, L)

    cos, sin = bd.rope_tables_flux(txt, hp, wp, HD, device=dev)
    gains = [torch.from_numpy(synth.gains(HD, 20 + i)).to(dev).bfloat16() for i in range(4)]

    def make_sets(seed, width, count):
        gen = torch.Generator(device=dev).manual_seed(seed)
        return [tuple(torch.randn(batch, L, width, device=dev, dtype=torch.bfloat16, generator=gen)
                      for _ in range(3)) for _ in range(count)]

    # Rotating input sets so that consecutive steps do not find their inputs in L2.
    set_bytes = 3 * batch * L * d_l * 2
    n_sets = max(2, int(np.ceil(160e6 / set_bytes)) + 1)
    sets = make_sets(1234 + rank, d_l, n_sets)
    kr = torch.empty(batch, L, d_l, device=dev, dtype=torch.bfloat16)
    # N > 1: the head outputs are gathered either by the attention kernel itself
    # (epilogue stores into every rank's replica through symmetric memory) or,
    # with --gather nccl, by an in-place NCCL all-gather of a head-major staging tensor.
    gathered, peer_ptrs, mc_ptrs = None, None, None
    gather_path = "none" if world == 1 else "nccl all-gather"
    config = workload_config(args, world)
    if world > 1 and args.gather.startswith("fused"):
        try:
            gathered = headshard.GatheredOutput(batch, L, NH, HD, torch.bfloat16, dev)
            peer_ptrs = [gathered.peer_ptrs(0), gathered.peer_ptrs(txt)]
            gather_path = "plain stores to every peer"
            # every rank must take the same path: the multicast address is used only if all have one
            have_mc = torch.tensor([1 if gathered.multicast_ptr(0) else 0], device=dev, dtype=torch.int32)
            dist.all_reduce(have_mc, op=dist.ReduceOp.MIN)
            if args.gather == "fused" and int(have_mc.item()) == 1:
                mc_ptrs = [gathered.multicast_ptr(0), gathered.multicast_ptr(txt)]
                peer_ptrs = None
                gather_path = "multimem.st to the switch's multicast address"
        except Exception as e:      # symmetric memory unavailable: NCCL path
            gathered, peer_ptrs, mc_ptrs = None, None, None
            gather_path = f"nccl all-gather (symmetric memory unavailable: {type(e).__name__})"
    staging = torch.empty(headshard.staging_shape(world, batch, L, NH, HD), device=dev,
                          dtype=torch.bfloat16)
    out = gathered.local if gathered is not None else staging[rank]

    # RMSNorm + RoPE of K is a pre-pass (every query-tile CTA of a head re-reads K).
    # RMSNorm + RoPE of Q: --q-norm fused = by the attention kernel on its own query
    # tiles; --q-norm prepass = two more jobs of the pre-pass launch.
    q_fused = args.q_norm == "fused"
    qr = None if q_fused else torch.empty(batch, L, d_l, device=dev, dtype=torch.bfloat16)

    def norm_rope(q, k, kr_=None, qr_=None, heads=None):
        kr_ = kr if kr_ is None else kr_
        qr_ = qr if qr_ is None else qr_
        jobs = []
        for b in range(batch):
            jobs += [
                dict(x=k[b, :txt], out=kr_[b, :txt], gain=gains[3], cos=cos, sin=sin, rope_row0=0),
                dict(x=k[b, txt:], out=kr_[b, txt:], gain=gains[1], cos=cos, sin=sin, rope_row0=txt),
            ]
            if not q_fused:
                jobs += [dict(x=q[b, :txt], out=qr_[b, :txt], gain=gains[2], cos=cos, sin=sin, rope_row0=0),
                         dict(x=q[b, txt:], out=qr_[b, txt:], gain=gains[0], cos=cos, sin=sin, rope_row0=txt)]
        for j0 in range(0, len(jobs), 4):       # one launch takes up to four (segment, batch item) jobs
            bd.rmsnorm_rope(jobs[j0:j0 + 4], nh_l if heads is None else heads, HD)

    q_norm = dict(gain=[gains[2], gains[0]], cos=cos, sin=sin, rope_row0=0) if q_fused else {}

    def attention(q, v, out_=None, kr_=None, qr_=None, heads=None, peers=True):
        out_ = out if out_ is None else out_
        kr_ = kr if kr_ is None else kr_
        qq = q if q_fused else (qr if qr_ is None else qr_)
        bd.sdpa_fwd([qq[:, :txt], qq[:, txt:]], [kr_[:, :txt], kr_[:, txt:]], [v[:, :txt], v[:, txt:]],
                    [out_[:, :txt], out_[:, txt:]], nh_l if heads is None else heads, q_norm=q_norm,
                    peer_out_ptrs=peer_ptrs if peers else None,
                    multicast_out_ptrs=mc_ptrs if peers else None)

    def gather():
        if gathered is not None:
            gathered.barrier()
        elif world > 1:
            headshard.all_gather_heads(staging)

    launches_per_step = -(-(batch * (2 if q_fused else 4)) // 4) + 1

    def step(i):
        q, k, v = sets[i % n_sets]
        norm_rope(q, k)
        attention(q, v)
        gather()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def check_status(where):
        """A device-side failure on any rank ends the run on every rank at the same point:
        all of them finish their streams, leave the process group together and only then
        raise, so that no rank goes away while the others still run kernels that store
        through the multicast object its memory is bound to."""
        bad = 1 if bd.device_status() != 0 else 0
        if world > 1:
            t = torch.tensor([bad], device=dev, dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            bad = int(t.item())
        if bad:
            if world > 1:
                torch.cuda.synchronize()
                dist.barrier()
                dist.destroy_process_group()
            raise RuntimeError(f"a kernel reported a device-side failure {where}")

    def check_gather():
        """One more step on set 0, then rank 0 recomputes the heads rank 1 owns from
        rank 1's own inputs (regenerated from its seed) with the plain, unsharded launch
        and compares them bit for bit with its gathered copy.  Every rank gets the result."""
        step(0)
        barrier()
        flag = torch.zeros(1, device=dev, dtype=torch.int32)
        if rank == 0:
            oq, ok_, ov = make_sets(1234 + 1, d_l, 1)[0]
            o_kr, o_qr = torch.empty_like(ok_), (None if q_fused else torch.empty_like(oq))
            o_out = torch.empty_like(oq)
            norm_rope(oq, ok_, kr_=o_kr, qr_=o_qr)
            attention(oq, ov, out_=o_out, kr_=o_kr, qr_=o_qr, peers=False)
            torch.cuda.synchronize()
            c0 = headshard.head_range(NH, world, 1)[0] * HD
            theirs = gathered.full[:, :, c0:c0 + d_l] if gathered is not None else staging[1]
            same = torch.equal(theirs, o_out)
            # and this rank's own columns of its own copy (they too arrive through the gather)
            mq, mk, mv = sets[0]
            norm_rope(mq, mk, kr_=o_kr, qr_=o_qr)
            attention(mq, mv, out_=o_out, kr_=o_kr, qr_=o_qr, peers=False)
            torch.cuda.synchronize()
            mine = gathered.full[:, :, :d_l] if gathered is not None else staging[0]
            same = same and torch.equal(mine, o_out)
            flag[0] = 1 if same else 0
            del oq, ok_, ov, o_kr, o_qr, o_out
        dist.broadcast(flag, src=0)
        barrier()
        return "bit-exact" if int(flag.item()) == 1 else "mismatch"

    for i in range(args.warmup):
        step(i)
    barrier()
    check_status("during warm-up")
    def time_attention_kernel(iters):
        """Average device time of the attention launch alone (events on the launching stream)."""
        ke = [torch.cuda.Event(enable_timing=True) for _ in range(2 * iters)]
        for i in range(iters):
            qq, _, vv = sets[i % n_sets]
            ke[2 * i].record()
            attention(qq, vv)
            ke[2 * i + 1].record()
        torch.cuda.synchronize()
        return sum(ke[2 * i].elapsed_time(ke[2 * i + 1]) for i in range(iters)) / iters

    # The dominant kernel timed alone, before the long timed region: this is the
    # state the burst cuBLAS peak was measured in.  (It is timed again after the
    # timed region, in the sustained power state, against the sustained peak.)
    q, k, v = sets[0]
    norm_rope(q, k)
    torch.cuda.synchronize()
    kernel_ms = time_attention_kernel(10)
    # the same launch without the query RMSNorm + RoPE prologue (queries normalised
    # beforehand): the tensor-bound main loop alone
    qn_saved = dict(q_norm)
    q_norm.clear()
    kernel_ms_plain = time_attention_kernel(10)
    q_norm.update(qn_saved)
    barrier()

    # ------------------------------------------------------- the timed regions
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    region_ms = []
    barrier()
    sampler.start()
    for _ in range(args.repeats):
        barrier()
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        barrier()
        region_ms.append(e0.elapsed_time(e1) / args.steps)
    sampler.stop()
    if world > 1:
        t = torch.tensor(region_ms, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        region_ms = [float(x) for x in t.tolist()]
    ms = statistics.median(region_ms)
    check_status("during the timed region")

    # the same kernel again, now in the sustained power state
    q, k, v = sets[0]
    norm_rope(q, k)
    torch.cuda.synchronize()
    kernel_ms_sustained = time_attention_kernel(max(5, min(50, args.steps)))
    peak_tf, peak_gbs, peak_kind = measured_peaks()
    local_flops = flops * nh_l / NH
    achieved = local_flops / (kernel_ms * 1e-3) / 1e12
    achieved_sustained = local_flops / (kernel_ms_sustained * 1e-3) / 1e12

    # ------------------------------------------------ N > 1: gather check, 1-GPU figure
    gather_check, one_gpu = None, None
    if world > 1:
        gather_check = check_gather()
        barrier()
        # rank 0 alone on the whole call (all 24 heads, no gather), for a like-for-like
        # scaling figure; the other ranks wait at the barrier
        if rank == 0:
            f_sets = make_sets(4321, D, 2)
            f_kr = torch.empty(batch, L, D, device=dev, dtype=torch.bfloat16)
            f_qr = None if q_fused else torch.empty_like(f_kr)
            f_out = torch.empty_like(f_kr)

            def full_step(i):
                fq, fk, fv = f_sets[i % 2]
                norm_rope(fq, fk, kr_=f_kr, qr_=f_qr, heads=NH)
                attention(fq, fv, out_=f_out, kr_=f_kr, qr_=f_qr, heads=NH, peers=False)

            for i in range(3):
                full_step(i)
            torch.cuda.synchronize()
            n1 = 10
            e0.record()
            for i in range(n1):
                full_step(i)
            e1.record()
            torch.cuda.synchronize()
            ms1 = e0.elapsed_time(e1) / n1
            v1 = flops / (ms1 * 1e-3) / 1e12
            one_gpu = {"ms_per_step": ms1, "value": v1, "unit": "TFLOP/s", "steps": n1,
                       "what": "rank 0 alone: all 24 heads of the same call, no gather, other ranks idle",
                       "efficiency_vs_it": (flops / (ms * 1e-3) / 1e12) / (world * v1)}
            del f_sets, f_kr, f_qr, f_out
        barrier()

    # ------------------------------------------------------------ end to end
    # host buffers in, result back to the host, every step
    hq, hk, hv = (torch.randn(batch, L, d_l, dtype=torch.bfloat16).pin_memory() for _ in range(3))
    ho = torch.empty(batch, L, d_l, dtype=torch.bfloat16).pin_memory()
    # K and V go up first, then the query rows in chunks; each chunk is normalised,
    # rotated and attended as soon as it has arrived (query rows are independent), and
    # its output rows go back to the host while the next chunk is computed, so the two
    # PCIe directions and the kernels overlap.  Two sets of device buffers alternate so
    # that step i+1 can start uploading while step i drains.  With N > 1 every rank
    # runs this pipeline on its own heads; the chunks of one step share one cross-GPU
    # barrier after the last chunk (fused gather) or one NCCL all-gather.
    e2e_mode = "pipelined: K/V upload, then query-row chunks over upload / compute / download streams"
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def buf():
        return torch.empty(batch, L, d_l, device=dev, dtype=torch.bfloat16)

    bufs = [dict(q=buf(), k=buf(), v=buf(), kr=buf(), done=None, drained=None) for _ in range(2)]
    for Bf in bufs:
        Bf["o"] = out if world > 1 else buf()
        Bf["od"] = buf() if world > 1 else None
    img = L - txt
    n_img_chunks = 4 if img % 4 == 0 and (img // 4) % 256 == 0 else 1
    chunks = [(0, txt)] + [(txt + c * (img // n_img_chunks), txt + (c + 1) * (img // n_img_chunks))
                           for c in range(n_img_chunks)]
    step_no = [0]

    def e2e_step():
        Bf = bufs[step_no[0] % 2]
        step_no[0] += 1
        cur = torch.cuda.current_stream(dev)
        if Bf["done"] is not None:
            s_in.wait_event(Bf["done"])        # the kernels that read this buffer set two steps ago
        with torch.cuda.stream(s_in):
            Bf["k"].copy_(hk, non_blocking=True)
            Bf["v"].copy_(hv, non_blocking=True)
            ev_kv = torch.cuda.Event()
            ev_kv.record(s_in)
            ev_q = []
            for r0, r1 in chunks:
                for b in range(batch):             # one contiguous slab per copy
                    Bf["q"][b, r0:r1].copy_(hq[b, r0:r1], non_blocking=True)
                e = torch.cuda.Event()
                e.record(s_in)
                ev_q.append(e)
        cur.wait_event(ev_kv)
        # this set's output buffer has reached the host (with N > 1 both sets write
        # the one gathered output, so the previous step's download is the one to wait for)
        prev = bufs[(step_no[0]) % 2]["drained"] if world > 1 else Bf["drained"]
        for ev in (Bf["drained"], prev):
            if ev is not None:
                cur.wait_event(ev)
        for b in range(batch):
            bd.rmsnorm_rope([
                dict(x=Bf["k"][b, :txt], out=Bf["kr"][b, :txt], gain=gains[3], cos=cos, sin=sin, rope_row0=0),
                dict(x=Bf["k"][b, txt:], out=Bf["kr"][b, txt:], gain=gains[1], cos=cos, sin=sin, rope_row0=txt),
            ], nh_l, HD)
        for ci, (r0, r1) in enumerate(chunks):
            cur.wait_event(ev_q[ci])
            pp, mp = None, None
            if gathered is not None:                 # the same gather form as the timed region
                if mc_ptrs is not None:
                    mp = [gathered.multicast_ptr(r0)]
                else:
                    pp = [gathered.peer_ptrs(r0)]
            bd.sdpa_fwd(Bf["q"][:, r0:r1], [Bf["kr"][:, :txt], Bf["kr"][:, txt:]],
                        [Bf["v"][:, :txt], Bf["v"][:, txt:]], Bf["o"][:, r0:r1], nh_l,
                        q_norm=dict(gain=gains[2] if r0 < txt else gains[0], cos=cos, sin=sin, rope_row0=r0),
                        peer_out_ptrs=pp, multicast_out_ptrs=mp)
            ev_o = torch.cuda.Event()
            ev_o.record(cur)
            s_out.wait_event(ev_o)
            with torch.cuda.stream(s_out):
                for b in range(batch):
                    if world == 1:
                        ho[b, r0:r1].copy_(Bf["o"][b, r0:r1], non_blocking=True)
                    else:
                        # rows of the gathered output are D wide: gather this rank's head
                        # columns into a dense slab first, then one contiguous download
                        Bf["od"][b, r0:r1].copy_(Bf["o"][b, r0:r1], non_blocking=True)
                        ho[b, r0:r1].copy_(Bf["od"][b, r0:r1], non_blocking=True)
        gather()
        Bf["done"] = torch.cuda.Event()
        Bf["done"].record(cur)
        Bf["drained"] = torch.cuda.Event()
        Bf["drained"].record(s_out)

    def e2e_join():
        cur = torch.cuda.current_stream(dev)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_join()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    check_status("during the end-to-end region")

    if rank == 0:
        line = {
            "metric": "attention TFLOP/s", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "repeats": args.repeats,
            "ms_per_step": ms, "ms_per_step_min": min(region_ms), "ms_per_step_max": max(region_ms),
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "l2_sets": f"{n_sets} input sets, {n_sets * set_bytes / 1e6:.0f} MB per rank",
            "clocks": sampler.summary(),
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": e2e_ms, "mode": e2e_mode, "host_cores": host_binding,
                    "h2d_bytes_per_step": 3 * batch * L * d_l * 2,
                    "d2h_bytes_per_step": batch * L * d_l * 2},
            "gpu_launches": launches_per_step * args.steps * args.repeats,
            "roofline": {"bound": "tensor", "kernel": "sdpa_tc05_kernel", "achieved": achieved,
                         "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "peak_kind": f"{peak_kind} cuBLAS bf16 burst", "kernel_ms": kernel_ms,
                         "frac_of_nominal_2250": achieved / 2250.0,
                         # achieved / frac: the kernel timed alone before the timed region,
                         # against the burst cuBLAS figure; *_sustained: timed again in a
                         # back-to-back loop after it, against the sustained cuBLAS figure
                         "achieved_sustained": achieved_sustained, "kernel_ms_sustained": kernel_ms_sustained,
                         # with --q-norm fused the launch above normalises and rotates its
                         # query tiles first; *_plain is the kernel given pre-normalised queries
                         "kernel_ms_plain": kernel_ms_plain,
                         "achieved_plain": local_flops / (kernel_ms_plain * 1e-3) / 1e12,
                         "frac_plain": local_flops / (kernel_ms_plain * 1e-3) / 1e12 / peak_tf,
                         "peak_sustained": sustained_peak_tf(),
                         "frac_of_sustained": achieved_sustained / sustained_peak_tf(),
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload)},
        }
        if world > 1:
            line["gather_check"] = gather_check
            line["gather_path"] = gather_path
            line["one_gpu_same_workload"] = one_gpu
        if world == 1:
            if not args.no_also:
                line["library_baseline"] = library_baselines(sets, batch, L, nh_l)
                line["also"] = other_configurations(bd)
                if bd.device_status() != 0:
                    raise RuntimeError("a kernel reported a device-side failure in the other configurations")
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline(L)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
        if rank == 0 and gather_check != "bit-exact":
            raise SystemExit(f"gathered head outputs differ from the locally recomputed ones ({gather_check})")


def run_sana(args):
    """Sana 1600M linear attention on one GPU: one step = one bdattn_linear_attn_relu_fwd call on a
    (batch, 2240, tokens) channel-major BF16 problem; metric = algorithmic GB/s
    (4 * tokens * 2240 * 2 bytes per batch item).  Steps are replayed from a
    CUDA graph so that host launch gaps do not enter the device time."""
    import torch
    import brodiffusion_b200 as bd
    torch.cuda.set_device(0)
    B, nh, N = SANA_WORKLOADS[args.workload]
    sampler = ClockSampler(0)
    ms, gbs, n_sets, byt = measure_sana(bd, B, nh, N, steps=args.steps, sampler=sampler)
    if bd.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side failure")
    _, peak_gbs, kind = measured_peaks()
    line = {"metric": "linear-attention GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "batch": B, "heads": nh, "head_dim": 32, "tokens": N,
                       "l2": f"rotating {n_sets} input sets ({n_sets * byt / 1e6:.0f} MB > 126 MB L2)",
                       "timing": "CUDA-graph replay of the steps, median of 5"},
            "clocks": sampler.summary(), "gpu_launches": args.steps * 5,
            "roofline": {"bound": "hbm", "kernel": "linear_attn_kernel", "achieved": gbs, "peak": peak_gbs,
                         "unit": "GB/s", "frac": gbs / peak_gbs, "peak_kind": f"{kind} copy bandwidth",
                         "traffic": None}}
    print(json.dumps(line), flush=True)


def run_proj(args):
    """Projections around the Flux 1024 px attention call on one GPU
    (4608 tokens, 3072 -> 3072 features, BF16): flux1024_qkv_proj = one
    bdattn_qkv_norm_rope_fwd call (Q, K and V projections with per-head RMSNorm
    and RoPE in the epilogue), flux1024_out_proj = one bdattn_linear_fwd call.
    metric = projection TFLOP/s (2 * tokens * in * out per projection).  Steps
    are replayed from a CUDA graph; activations rotate over sets larger than L2."""
    import torch
    import brodiffusion_b200 as bd
    torch.cuda.set_device(0)
    n_proj = PROJ_WORKLOADS[args.workload]
    sampler = ClockSampler(0)
    ms, tf = measure_proj(bd, n_proj, steps=args.steps, sampler=sampler)
    if bd.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side failure")
    peak_tf, _, kind = measured_peaks()
    line = {"metric": "projection TFLOP/s", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "tokens": 4608, "in_features": 3072, "out_features": 3072,
                       "projections": n_proj, "heads": 24, "head_dim": 128,
                       "l2": "rotating 6 activation sets (170 MB > 126 MB L2)",
                       "timing": "CUDA-graph replay of the steps, median of 5"},
            "clocks": sampler.summary(), "gpu_launches": args.steps * 5,
            "roofline": {"bound": "tensor", "kernel": "gemm_wide_kernel", "achieved": tf, "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": tf / peak_tf, "peak_kind": f"{kind} cuBLAS BF16 burst",
                         "traffic": None}}
    print(json.dumps(line), flush=True)


def cpu_baseline(L):
    """Oracle port of the reference attention core on the host cores, on a
    bounded sample of the same workload (about 10-20 s of CPU work)."""
    import numpy as np
    import synth
    from oracle import oracle as O
    O.build()
    cores = O.hardware_threads()
    q = synth.activations((L, D), 11)
    k = synth.activations((L, D), 12)
    v = synth.activations((L, D), 13)
    probe = np.arange(0, L, L // 16, dtype=np.int32)[:16]
    t0 = time.perf_counter()
    O.sdpa(q, k, v, NH, rows=probe, precise=False)
    per_row = (time.perf_counter() - t0) / len(probe)
    rows_n = int(max(16, min(L, 12.0 / per_row)))
    rows = np.linspace(0, L - 1, rows_n).astype(np.int32)
    t0 = time.perf_counter()
    O.sdpa(q, k, v, NH, rows=rows, precise=False)
    dt = time.perf_counter() - t0
    return {"value": 4.0 * rows_n * L * D / dt / 1e12, "unit": "TFLOP/s", "cores": cores,
            "kind": "port",
            "sample": f"{rows_n} of {L} query rows (all {NH} heads, all keys), attention core "
                      f"FP32, {dt:.1f} s; full call extrapolates to {L / rows_n * dt:.1f} s"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=30,
                    help="how many times the K-step timed region is measured (median reported)")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + sorted(SANA_WORKLOADS) + sorted(PROJ_WORKLOADS),
                    default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true",
                    help="skip the other configurations and the library baselines (1 GPU)")
    ap.add_argument("--q-norm", choices=["fused", "prepass"], default=None,
                    help="RMSNorm + RoPE of Q inside the attention kernel or in the pre-pass")
    ap.add_argument("--gather", choices=["fused", "fused-peer", "nccl"], default="fused",
                    help="N > 1: how the head outputs are gathered")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload is None:
        args.workload = "flux1024" if max(world, args.gpus) == 1 else "flux2048_headsharded"
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    if args.q_norm is None:
        args.q_norm = "prepass"
    if args.workload in SANA_WORKLOADS:
        if args.impl == "reference" or world > 1:
            raise SystemExit("the sana workloads run on one GPU with --impl ours")
        run_sana(args)
        return
    if args.workload in PROJ_WORKLOADS:
        if args.impl == "reference" or world > 1:
            raise SystemExit("the projection workloads run on one GPU with --impl ours")
        run_proj(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with "
                         "python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
