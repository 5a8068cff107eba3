"""RotorQuant (rust-nn src/quant.rs): `Rotor` (a Cl(3,0) rotor: scalar + three bivector parts) and
`RotorQuant(dim, bits)`, a fake-quantiser that rotates consecutive 3-groups of the last axis with
fixed random rotors, quantises each rotated group symmetrically to `bits` bits and rotates back.

The rotors come from a seeded generator (default seed 0xC11FC0DE as in the reference, whose
`StdRng` stream is not reproduced bit for bit). On CUDA tensors the whole rotate-quantise-rotate
runs as one kernel with one thread per (row, group).
"""
from __future__ import annotations

import math
import random
from typing import List

import torch

from . import nn
from .ops import quant_kernels as Q


class Rotor:
    def __init__(self, s: float, p12: float, p13: float, p23: float):
        self.s, self.p12, self.p13, self.p23 = s, p12, p13, p23

    @staticmethod
    def random(rng: random.Random) -> "Rotor":
        a, b, c = (rng.uniform(-1.0, 1.0) for _ in range(3))
        norm = math.sqrt(a * a + b * b + c * c)
        theta = rng.uniform(0.0, math.pi)
        if norm < 1e-8:
            return Rotor(1.0, 0.0, 0.0, 0.0)
        mag = math.sin(theta / 2.0)
        return Rotor(math.cos(theta / 2.0), mag * a / norm, mag * b / norm, mag * c / norm)

    @staticmethod
    def _apply(x, s, p12, p13, p23):
        return [
            s * x[0] - p12 * x[4] - p13 * x[5] - p23 * x[6],
            s * x[1] + p12 * x[2] + p13 * x[3] + p23 * x[7],
            s * x[2] - p12 * x[1] + p23 * x[3] - p13 * x[7],
            s * x[3] - p13 * x[1] - p23 * x[2] + p12 * x[7],
            s * x[4] + p12 * x[0],
            s * x[5] + p13 * x[0],
            s * x[6] + p23 * x[0],
            s * x[7] - p23 * x[1] + p13 * x[2] - p12 * x[3],
        ]

    def sandwich(self, x: List[float]) -> List[float]:
        """R x R~ on an 8-component multivector [1, e1, e2, e3, e12, e13, e23, e123]."""
        return self._apply(self._apply(x, self.s, self.p12, self.p13, self.p23), self.s, -self.p12, -self.p13, -self.p23)

    def inv_sandwich(self, x: List[float]) -> List[float]:
        return self._apply(self._apply(x, self.s, -self.p12, -self.p13, -self.p23), self.s, self.p12, self.p13, self.p23)

    def rotation_matrix(self) -> List[List[float]]:
        cols = []
        for k in range(3):
            e = [0.0] * 8
            e[1 + k] = 1.0
            cols.append(self.sandwich(e))
        return [[cols[j][1 + i] for j in range(3)] for i in range(3)]


class RotorQuant(nn.Module):
    DEFAULT_SEED = 0xC11FC0DE

    def __init__(self, dim: int, bits: int, seed: int = DEFAULT_SEED):
        if bits < 2:
            raise ValueError("RotorQuant needs at least 2 bits")
        self.dim, self.bits = dim, bits
        self.padded_dim = (dim + 2) // 3 * 3
        rng = random.Random(seed)
        self.rotors = [Rotor.random(rng) for _ in range(self.padded_dim // 3)]
        self._rot = torch.tensor([r.rotation_matrix() for r in self.rotors], dtype=torch.float32).reshape(-1, 9)

    @staticmethod
    def new(dim: int, bits: int) -> "RotorQuant":
        return RotorQuant(dim, bits)

    @staticmethod
    def with_seed(dim: int, bits: int, seed: int) -> "RotorQuant":
        return RotorQuant(dim, bits, seed)

    def qmax(self) -> float:
        return float((1 << (self.bits - 1)) - 1)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() == 0 or x.shape[-1] != self.dim:
            raise ValueError(f"RotorQuant configured for dim {self.dim} but got last-dim {x.shape[-1] if x.dim() else 0}")
        if self._rot.device != x.device:
            self._rot = self._rot.to(x.device)
        return Q.rotor_quant(x.detach(), self._rot, self.dim, self.qmax())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.quantize(x)

    def parameters(self):
        return []


from ._compat import install as _install  # noqa: E402

_install(globals())
