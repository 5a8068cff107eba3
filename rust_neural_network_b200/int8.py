"""INT8 inference (rust-nn src/int8.rs): `Int8Weights`, `Int8Linear`, `igemm`, `igemm_scalar`.

The integer product runs on the tensor cores (`tcgen05.mma.kind::i8`, int32 accumulators in TMEM);
dequantisation (row scale x column scale), bias and activation are the GEMM's epilogue.

Activation scaling. The reference quantises each activation with the scale of the WEIGHT row it is
about to meet (`a_q = round(x / w_scale[o])`, src/int8.rs:70-88, 134-165), which makes the quantised
activation depend on the output column and is therefore not a matrix product. `Int8Linear.forward`
uses the standard scheme instead - one dynamic symmetric scale per activation row - which is a real
int8 GEMM and is more accurate; `mode="reference"` evaluates the reference's formula exactly
(an O(M*N*K) elementwise evaluation, kept as the parity oracle).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import nn
from .ops import gemm as G
from .ops import quant_kernels as Q


class Int8Weights:
    """Per-row symmetric int8 weights: `data` int8 [out, in], `scales` fp32 [out], scale = max|row|/127."""

    def __init__(self, data: torch.Tensor, scales: torch.Tensor, shape):
        self.data, self.scales, self.shape = data, scales, list(shape)

    @staticmethod
    def quantize(weight: torch.Tensor) -> "Int8Weights":
        w = weight.detach()
        q, s = Q.quant_rows(w.reshape(w.shape[0], -1), "int8")
        return Int8Weights(q, s, w.shape)

    def dequantize(self) -> torch.Tensor:
        return (self.data.float() * self.scales[:, None]).reshape(self.shape)

    def matmul_f32(self, activation: torch.Tensor, m: Optional[int] = None, mode: str = "rowwise") -> torch.Tensor:
        """`activation` [m, in] (or flat with `m` rows) -> [m, out] fp32."""
        out_f, in_f = self.shape
        a = activation.reshape(-1, in_f) if m is None else activation.reshape(m, in_f)
        if mode == "reference":
            return _reference_formula(a, self)
        return _int8_linear(a, self, None, "none", torch.float32)

    def mem_bytes(self) -> int:
        return self.data.numel() + self.scales.numel() * 4

    def compression_ratio(self) -> float:
        return self.data.numel() * 4 / self.mem_bytes()

    def quantization_error(self, original: torch.Tensor) -> float:
        return float((original.detach().float().reshape(self.shape).to(self.data.device) - self.dequantize()).abs().mean())


def _reference_formula(a: torch.Tensor, w: Int8Weights) -> torch.Tensor:
    s = w.scales.float()
    aq = Q.round_away(a.float()[:, None, :] / s[None, :, None]).clamp(-128, 127)             # [m, out, in]
    acc = (aq * w.data.float()[None]).sum(-1)
    return acc * s * s


def _int8_linear(a: torch.Tensor, w: Int8Weights, bias, act: str, out_dtype) -> torch.Tensor:
    aq, a_scale = Q.quant_rows(a, "int8")
    return G.gemm(aq, w.data, row_scale=a_scale, col_scale=w.scales, bias=bias, act=act, out_dtype=out_dtype)


class Int8Linear(nn.Module):
    def __init__(self, int8_weight: Int8Weights, bias: Optional[torch.Tensor], mode: str = "rowwise"):
        self.int8_weight, self.bias, self.mode = int8_weight, bias, mode

    @staticmethod
    def from_linear(layer: nn.Linear, mode: str = "rowwise") -> "Int8Linear":
        b = layer.bias.detach().float().clone() if layer.bias is not None else None
        return Int8Linear(Int8Weights.quantize(layer.weight), b, mode)

    def forward(self, x: torch.Tensor, act: str = "none", out_dtype=torch.float32) -> torch.Tensor:
        in_f = x.shape[-1]
        a = x.detach().reshape(-1, in_f)
        if self.mode == "reference":
            y = _reference_formula(a, self.int8_weight)
            if self.bias is not None:
                y = y + self.bias
            y = G.act_ref(y, act).to(out_dtype)
        else:
            y = _int8_linear(a, self.int8_weight, self.bias, act, out_dtype)
        return y.reshape(*x.shape[:-1], self.int8_weight.shape[0])

    def parameters(self):
        return []


def igemm_scalar(a: torch.Tensor, b: torch.Tensor, m: int, k: int, n: int) -> torch.Tensor:
    """The scalar oracle: A uint8 [m, k], B int8 [k, n] -> int32 [m, n] (src/int8.rs:222-234)."""
    return (a.reshape(m, k).to(torch.int64).cpu() @ b.reshape(k, n).to(torch.int64).cpu()).to(torch.int32)


def igemm(a: torch.Tensor, b: torch.Tensor, m: int, k: int, n: int) -> torch.Tensor:
    """uint8 x int8 -> int32 on the tensor cores. `b` is [k, n] row-major as in the reference; the
    kernel wants it K-major, so it is transposed once here (weights should be stored [n, k])."""
    a2, b2 = a.reshape(m, k), b.reshape(k, n)
    if not a2.is_cuda:
        return igemm_scalar(a2, b2, m, k, n)
    return G.gemm(a2.contiguous(), b2.t().contiguous(), out_dtype=torch.int32)


from ._compat import install as _install  # noqa: E402

_install(globals())
