"""Shared test configuration.

``-m "not gpu"`` runs on any host (oracle vs golden fixtures, host-side logic,
C-ABI loading).  ``-m gpu`` tests need a B200: they call the CUDA kernels
through the C ABI and compare against the oracle; they fail (not skip) when
CUDA or the built library is missing.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "golden.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def bd():
    """The product binding with a CUDA device; fails loudly when absent."""
    import torch
    import brodiffusion_b200 as bd
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert os.path.exists(bd.lib_path()), "libbdattn.so is not built"
    torch.cuda.set_device(0)
    return bd


def bf16_from_bits(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def compare(got, ref):
    """max-abs error and cosine similarity of two arrays."""
    got = np.asarray(got, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    err = float(np.abs(got - ref).max())
    cos = float((got * ref).sum() / (np.sqrt((got * got).sum() * (ref * ref).sum()) + 1e-300))
    return err, cos
