"""`CompiledMLP` (rust-nn src/compiled.rs): an MLP whose whole training step - forward, mean-squared
error, backward, Adam - is fixed at construction time.

The reference pre-allocates every buffer and hand-fuses the backward to remove autograd overhead
(src/compiled.rs:90-300). The same idea here is a CUDA graph: the step (GEMMs with bias + ReLU in
their epilogues, the loss kernel, the backward GEMMs with the ReLU gate in their epilogues, fused
Adam) is recorded once on static buffers and replayed with a single launch. On a CPU tensor the
step runs eagerly. Initialisation follows the reference: weights from its LCG
(seed = in*31 + out; x <- 1664525 x + 1013904223; ((x >> 8) / 2^24 - 0.5) * 2 * sqrt(2/in)), zero
biases, ReLU on every layer but the last, Adam(0.9, 0.999, 1e-8).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from . import nn
from .loss import MSELoss
from .optim import Adam
from .train import Trainer


def _lcg_weights(lin: int, lout: int) -> torch.Tensor:
    n = lout * lin
    seed = (lin * 31 + lout) & 0xFFFFFFFF
    out = np.empty(n, dtype=np.float32)
    std = np.float32((2.0 / lin) ** 0.5)
    # x_{i+1} = a x_i + c (mod 2^32), vectorised by jumping: x_i = A_i x_0 + C_i
    a, c = 1664525, 1013904223
    A = np.empty(n, dtype=np.uint64); Cc = np.empty(n, dtype=np.uint64)
    ai, ci = 1, 0
    for i in range(n) if n <= 4096 else range(0):
        ai = (ai * a) & 0xFFFFFFFF; ci = (ci * a + c) & 0xFFFFFFFF
        A[i], Cc[i] = ai, ci
    if n > 4096:
        x = seed
        vals = np.empty(n, dtype=np.uint32)
        for i in range(n):
            x = (x * a + c) & 0xFFFFFFFF
            vals[i] = x
    else:
        vals = ((A * np.uint64(seed) + Cc) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    out[:] = ((vals >> 8).astype(np.float32) / np.float32(16777216.0) - np.float32(0.5)) * np.float32(2.0) * std
    return torch.from_numpy(out).reshape(lout, lin)


class CompiledMLP:
    def __init__(self, dims: Sequence[Tuple[int, int]], batch: int, lr: float, device=None, dtype=torch.float32):
        self.dims, self.batch, self.lr = [tuple(d) for d in dims], batch, lr
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.model = nn.Sequential()
        for i, (lin, lout) in enumerate(self.dims):
            layer = nn.Linear(lin, lout, True)
            layer.weight.data.copy_(_lcg_weights(lin, lout))
            self.model.add(layer)
            if i + 1 < len(self.dims):
                self.model.add(nn.ReLU())
        self.model.to_device(self.device, dtype=dtype) if self.device.type == "cuda" else None
        self.optimizer = Adam(self.model.parameters(), lr=lr)
        self.trainer = Trainer(self.model, self.optimizer, MSELoss("mean"), use_cuda_graph=self.device.type == "cuda")
        self.t = 0

    @staticmethod
    def new(dims: Sequence[Tuple[int, int]], batch: int, lr: float) -> "CompiledMLP":
        return CompiledMLP(dims, batch, lr)

    def _as_batch(self, v, width: int) -> torch.Tensor:
        t = v if isinstance(v, torch.Tensor) else torch.as_tensor(np.asarray(v, dtype=np.float32))
        return t.reshape(self.batch, width)

    def step_async(self, x, target) -> torch.Tensor:
        """One training step; returns the loss as a device tensor (no host sync)."""
        self.t += 1
        return self.trainer.train_step(self._as_batch(x, self.dims[0][0]), self._as_batch(target, self.dims[-1][1]))

    def step(self, x, target) -> float:
        return float(self.step_async(x, target))

    def forward(self, x) -> torch.Tensor:
        with torch.no_grad():
            t = self._as_batch(x, self.dims[0][0]).to(self.device)
            return self.model(t)

    def weights(self) -> List[torch.Tensor]:
        return [l.weight for l in self.model.layers if isinstance(l, nn.Linear)]

    def biases(self) -> List[torch.Tensor]:
        return [l.bias for l in self.model.layers if isinstance(l, nn.Linear)]


from ._compat import install as _install  # noqa: E402

_install(globals())
