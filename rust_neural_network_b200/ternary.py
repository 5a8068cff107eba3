"""Ternary (1.58-bit) weights (rust-nn src/ternary.rs): `TernaryTensor`, `TernaryLinear`,
`TernaryModel`, `ternarize`, `pack_ternary`, `unpack_ternary`.

Weights become {-1, 0, +1} * scale: threshold 0.7 * mean|w| and scale mean|w| per row, packed 16
codes to a 32-bit word (0 -> 0, +1 -> 1, -1 -> 2), low bits first (src/ternary.rs:46-137).
The reference's forward adds and subtracts activations in fp32 (src/ternary.rs:239-279). Here the
packed words stay the stored form; a kernel expands them to bf16 (in which {-1, 0, +1} are exact)
and the tensor-core GEMM multiplies, with the per-row scale and the bias applied in its epilogue.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import nn
from .ops import gemm as G
from .ops import quant_kernels as Q


def pack_ternary(values: Sequence[int]) -> List[int]:
    packed = [0] * ((len(values) + 15) // 16)
    for i, v in enumerate(values):
        code = 0 if v == 0 else (1 if v > 0 else 2)
        packed[i // 16] |= code << ((i % 16) * 2)
    return packed


def unpack_ternary(packed: Sequence[int], count: int) -> List[int]:
    out = []
    for i in range(count):
        code = (packed[i // 16] >> ((i % 16) * 2)) & 3
        out.append(1 if code == 1 else -1 if code == 2 else 0)
    return out


class TernaryTensor:
    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, shape, numel: int):
        self.packed, self.scales, self.shape, self.numel = packed, scales, list(shape), numel

    @property
    def cols(self) -> int:
        return self.shape[1] if len(self.shape) >= 2 else max(self.numel, 1)

    @staticmethod
    def quantize(tensor: torch.Tensor) -> "TernaryTensor":
        t = tensor.detach()
        numel = t.numel()
        rows = t.shape[0] if t.dim() >= 2 else 1
        cols = numel // max(rows, 1)           # trailing dims of an N-D tensor fold into the row
        packed, scales = Q.ternary_quant(t.reshape(rows, cols), rows, cols)
        return TernaryTensor(packed, scales, t.shape, numel)

    def values(self, out_dtype=torch.float32) -> torch.Tensor:
        """The unscaled codes as {-1, 0, +1}, in the tensor's shape."""
        return Q.ternary_unpack(self.packed, self.numel, self.cols, None, out_dtype).reshape(self.shape)

    def dequantize(self) -> torch.Tensor:
        return Q.ternary_unpack(self.packed, self.numel, self.cols, self.scales, torch.float32).reshape(self.shape)

    def mem_bytes(self) -> int:
        return self.packed.numel() * 4 + self.scales.numel() * 4

    def compression_ratio(self) -> float:
        return self.numel * 4 / max(self.mem_bytes(), 1)

    def quantization_error(self, original: torch.Tensor) -> float:
        o = original.detach().float().to(self.packed.device)
        return float((o - self.dequantize()).abs().sum() / max(o.numel(), 1))

    def value_counts(self):
        """(+1 count, -1 count, 0 count)."""
        return Q.ternary_counts(self.packed, self.numel)

    def sparsity(self) -> float:
        return self.value_counts()[2] / max(self.numel, 1)


class TernaryLinear(nn.Module):
    def __init__(self, ternary_weight: TernaryTensor, bias: Optional[torch.Tensor], in_features: int, out_features: int):
        self.ternary_weight, self.bias, self.in_features, self.out_features = ternary_weight, bias, in_features, out_features

    @staticmethod
    def from_linear(layer: nn.Linear) -> "TernaryLinear":
        b = layer.bias.detach().float().clone() if layer.bias is not None else None
        return TernaryLinear(TernaryTensor.quantize(layer.weight), b, layer.weight.shape[1], layer.weight.shape[0])

    def forward(self, x: torch.Tensor, act: str = "none", out_dtype=torch.float32) -> torch.Tensor:
        a = x.detach().reshape(-1, x.shape[-1])
        tw = self.ternary_weight
        if a.is_cuda:
            w = tw.values(torch.bfloat16).reshape(self.out_features, self.in_features)
            y = G.gemm(a.to(torch.bfloat16), w, col_scale=tw.scales, bias=self.bias, act=act, out_dtype=out_dtype)
        else:
            y = (a.float() @ tw.values().reshape(self.out_features, self.in_features).t()) * tw.scales
            if self.bias is not None:
                y = y + self.bias
            y = G.act_ref(y, act).to(out_dtype)
        return y.reshape(*x.shape[:-1], self.out_features)

    def parameters(self):
        return []


class TernaryModel:
    """Every 2-D parameter becomes a `TernaryLinear`; a following 1-D parameter is its bias (src/ternary.rs:292-329)."""

    def __init__(self, layers: List[TernaryLinear]):
        self.layers = layers

    @staticmethod
    def from_model(model) -> "TernaryModel":
        params = list(model.parameters())
        layers, i = [], 0
        while i < len(params):
            w = params[i]
            b = params[i + 1] if (i + 1 < len(params) and params[i + 1].dim() == 1) else None
            out_f = w.shape[0] if w.dim() >= 1 else 0
            in_f = w.shape[1] if w.dim() >= 2 else 0
            layers.append(TernaryLinear(TernaryTensor.quantize(w), b.detach().float().clone() if b is not None else None, in_f, out_f))
            i += 2 if b is not None else 1
        return TernaryModel(layers)

    def mem_bytes(self) -> int:
        return sum(l.ternary_weight.mem_bytes() + (l.bias.numel() * 4 if l.bias is not None else 0) for l in self.layers)

    def compression_ratio(self) -> float:
        return sum(l.ternary_weight.numel for l in self.layers) * 4 / max(self.mem_bytes(), 1)

    def avg_sparsity(self) -> float:
        if not self.layers:
            return 0.0
        return sum(l.ternary_weight.sparsity() for l in self.layers) / len(self.layers)

    def forward_first_layer(self, x: torch.Tensor) -> torch.Tensor:
        return self.layers[0].forward(x)

    def forward(self, x: torch.Tensor, activation: str = "relu") -> torch.Tensor:
        h = x
        for i, l in enumerate(self.layers):
            h = l.forward(h, act=activation if i + 1 < len(self.layers) else "none")
        return h


def ternarize(tensor: torch.Tensor) -> TernaryTensor:
    return TernaryTensor.quantize(tensor)


from ._compat import install as _install  # noqa: E402

_install(globals())
