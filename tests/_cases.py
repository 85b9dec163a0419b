"""Seeded synthetic inputs shared by the parity tests, the golden generator and bench.py.

The distributions follow the benchmark configurations of this repository:
activations N(0,1) with 1 % of input channels scaled x20 (outliers), weights
N(0,0.02), bias N(0,0.01); the reference smoke-test case uses plain randn
(tests/test_vdm_w4a4_kernel_smoke.py:15-23 of the reference).  Everything is
drawn from a CPU torch.Generator so every machine sees the same bits, then
rounded to fp16 once: CPU oracle and GPU kernels consume the same fp16 values.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(a)
        h.update(str(a.dtype).encode())
        h.update(str(a.shape).encode())
        h.update(a.tobytes())
    return h.hexdigest()


def make_case(seed: int, M: int, K: int, N: int, *, outliers: bool = True, w_std: float = 0.02,
              b_std: float = 0.01, bias: bool = True):
    """Returns fp16 numpy arrays x [M,K], w [N,K], b [N] (or None)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    if outliers:
        idx = torch.randperm(K, generator=g)[: max(1, K // 100)]
        x[:, idx] *= 20.0
    w = torch.randn(N, K, generator=g, dtype=torch.float32) * w_std
    b = torch.randn(N, generator=g, dtype=torch.float32) * b_std if bias else None
    x16 = x.half().numpy()
    w16 = w.half().numpy()
    b16 = b.half().numpy() if b is not None else None
    return x16, w16, b16


# name -> (seed, M, K, N, kwargs, clip)
CASES = {
    # Small enough to store every array in the fixture.
    "tiny": (7, 37, 128, 128, {}, 1.0),
    "tiny_clip": (8, 70, 192, 256, {}, 0.95),
    # BASELINE config 0: one QuantLinear, M=4096, K=N=1536, seed 0.
    "cfg0": (0, 4096, 1536, 1536, {}, 1.0),
    # Shape/seed/clip of the reference's kernel smoke test (plain randn inputs).
    "smoke257": (0, 257, 1536, 1536, {"outliers": False, "w_std": 1.0, "b_std": 1.0}, 0.95),
}
