"""Deterministic test-data generator.

Same recurrence and mapping as the generator the reference's kernel tests use
(rust-nn src/blas.rs:1182-1190): x <- 1664525*x + 1013904223 (mod 2^32), value = top 24 bits / 2^24 - 0.5,
so golden vectors can be shared between the two code bases. Vectorised with numpy.
"""
from __future__ import annotations

import numpy as np
import torch

_A = 1664525
_C = 1013904223


_TABLES = None


def _tables(chunk: int):
    global _TABLES
    if _TABLES is None:
        a_pow = np.empty(chunk, dtype=np.uint64)
        c_sum = np.empty(chunk, dtype=np.uint64)
        ap, cs = 1, 0
        for i in range(chunk):
            ap = (ap * _A) & 0xFFFFFFFF
            cs = (cs * _A + _C) & 0xFFFFFFFF
            a_pow[i] = ap
            c_sum[i] = cs
        _TABLES = (a_pow, c_sum)
    return _TABLES


def lcg_values(n: int, seed: int = 1) -> np.ndarray:
    """n values in [-0.5, 0.5), fp32."""
    # closed form of the affine recurrence: x_k = A^k x_0 + C (A^k - 1)/(A - 1)  (mod 2^32),
    # evaluated with prefix products in uint64 arithmetic chunk by chunk.
    out = np.empty(n, dtype=np.float32)
    x = np.uint64(seed & 0xFFFFFFFF)
    mask = np.uint64(0xFFFFFFFF)
    chunk = 1 << 16
    # per-chunk: powers of A and running sums of C*A^j
    a_pow, c_sum = _tables(chunk)
    pos = 0
    while pos < n:
        m = min(chunk, n - pos)
        xs = (a_pow[:m] * x + c_sum[:m]) & mask
        out[pos:pos + m] = (xs >> np.uint64(8)).astype(np.float32) / np.float32(16777216.0) - np.float32(0.5)
        x = xs[m - 1]
        pos += m
    return out


_CACHE: dict = {}


def lcg_tensor(shape, seed: int = 1) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    key = (n, seed)
    if key not in _CACHE:
        _CACHE[key] = torch.from_numpy(lcg_values(n, seed).copy())
        if len(_CACHE) > 64:
            _CACHE.pop(next(iter(_CACHE)))
    return _CACHE[key].clone().view(*shape)
