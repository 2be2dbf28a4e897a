"""Seeded synthetic inputs for the parity tests and the bench.

A counter-based generator (splitmix64, the same mixer the reference's CLI uses
for its synthetic latents, cli/cmd_model_fwd.cpp:827-841) so that any consumer
reproduces identical bits from (seed, size) alone.  Normals come from
Box-Muller on two uniform streams.  Values are rounded once to the storage
type so that the GPU and the CPU oracle consume identical numbers (the
pattern of tests/test_fused_parity.cpp:50-62).
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(counter: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = counter * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def uniform01(n: int, seed: int) -> np.ndarray:
    """n doubles in (0, 1), stream `seed`."""
    with np.errstate(over="ignore"):
        ctr = np.arange(1, n + 1, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x100000001B3)
    z = _splitmix64(ctr)
    return ((z >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def normal(shape, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    u1 = uniform01(n, 2 * seed + 1)
    u2 = uniform01(n, 2 * seed + 2)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).astype(np.float32).reshape(shape)


def round_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)


def round_fp16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def activations(shape, seed, dtype="bf16"):
    """N(0, 1), rounded to the storage type."""
    x = normal(shape, seed)
    return round_bf16(x) if dtype == "bf16" else round_fp16(x) if dtype == "fp16" else x


def weights(shape, seed, dtype="bf16"):
    """N(0, 0.02), rounded to the storage type."""
    x = normal(shape, seed, 0.0, 0.02)
    return round_bf16(x) if dtype == "bf16" else round_fp16(x) if dtype == "fp16" else x


def gains(n, seed, dtype="bf16"):
    """RMSNorm gains 1 + N(0, 0.02)."""
    x = normal((n,), seed, 1.0, 0.02)
    return round_bf16(x) if dtype == "bf16" else x
