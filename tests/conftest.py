"""Shared test helpers.

Markers: ``gpu`` - needs a CUDA device (B200); everything else runs on CPU.
The CPU oracle (package ``oracle``) is imported here and in the tests only.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA GPU (run with -m gpu on a B200)")


def make_activations(M, K, seed=0, outliers=8, outlier_gain=20.0):
    """fp16 [M,K] ~ N(0,1) with `outliers` seeded channels scaled by `outlier_gain`
    (stand-in for LLM activation outliers; the distribution the bench uses)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    if outliers and K >= outliers:
        cols = torch.randperm(K, generator=g)[:outliers]
        x[:, cols] *= outlier_gain
    return x.to(torch.float16).numpy()


def make_weight(N, K, seed=1, std=0.02):
    """fp16-rounded float32 weight [N,K] ~ N(0, std)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g, dtype=torch.float32) * std
    return w.to(torch.float16).to(torch.float32).numpy()


def rel_err(y, ref):
    """max |y-ref| / max |ref| (normalised max error) in float64."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    den = np.abs(ref).max()
    return float(np.abs(y - ref).max() / (den if den > 0 else 1.0))


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.lib()
    return o
