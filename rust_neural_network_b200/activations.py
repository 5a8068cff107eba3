"""Functional activations (rust-nn src/activations.rs): `relu`, `sigmoid`, `tanh`, `softmax`, `gelu`.
All five are differentiable here (the reference's tanh / softmax / gelu are forward-only) and run
as this package's elementwise kernels; softmax is over the last axis."""
import torch

from .ops import functional as F


def relu(x): return F.relu(x)
def sigmoid(x): return F.sigmoid(x)
def tanh(x): return F.tanh(x)
def gelu(x): return F.gelu(x)


def softmax(x):
    if x.dim() == 0:
        return torch.ones(1, dtype=x.dtype, device=x.device)
    if x.shape[-1] == 0:
        return x
    return F.softmax(x)


from ._compat import install as _install  # noqa: E402

_install(globals())
