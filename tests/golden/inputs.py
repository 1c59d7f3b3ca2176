"""Seeded synthetic inputs shared by the golden-vector generator and the tests.

Everything is drawn from torch's CPU generator with an explicit seed, so the
generator script (run where the reference is installed) and the tests (run
anywhere) see the same tensors; each golden file stores a SHA-256 of its inputs
and the tests compare it before trusting the stored outputs.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

# name -> (M tokens, K in_features, N out_features, seed)
CASES = {
    # BASELINE config 1: SmolLM2-135M MLP up-projection, seed 0
    "c1": (16, 576, 1536, 0),
    "k64": (3, 64, 32, 11),
    "k128": (1, 128, 48, 12),
    "k192": (5, 192, 80, 13),
    "k512": (8, 512, 128, 14),
    "k1024": (2, 1024, 64, 15),
}
# shapes whose K is a multiple of 128 also go through the reference's I2_S CPU kernel
I2S_CASES = ["k128", "k512", "k1024"]


def make_inputs(name: str):
    """Returns (x fp32 [M,K] ~ N(0,1), w fp32 [N,K] ~ N(0,0.02)) as torch CPU tensors."""
    m, k, n, seed = CASES[name]
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
    x = torch.randn(m, k, generator=g, dtype=torch.float32)
    return x, w


def with_outliers(x: torch.Tensor, seed: int, frac: float = 1e-3, mag: float = 20.0) -> torch.Tensor:
    """Activation distribution of the decode/prefill sweeps: N(0,1) with a `frac`
    share of entries replaced by +-mag."""
    g = torch.Generator().manual_seed(seed + 7919)
    mask = torch.rand(x.shape, generator=g) < frac
    sign = torch.where(torch.rand(x.shape, generator=g) < 0.5, -1.0, 1.0)
    return torch.where(mask, sign * mag, x)


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()
