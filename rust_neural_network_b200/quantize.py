"""Weight quantisation formats (rust-nn src/quantize.rs): `QuantFormat`, `QuantizedTensor`,
`QuantizedLinear`, `QuantizedModel`, `quantize`.

Formats, scales, lookup tables and nibble order follow the reference (INT8 max/127, INT4 max/7,
NF4 table with scale max, NVFP4 E2M1 magnitudes with scale max/6, Q4_0 blocks of <=32 with the
negative scale max/-8, Q8_0 blocks of <=32; low nibble first). Quantise / dequantise run as CUDA
kernels on device tensors. FP16 / BF16 use the hardware's round-to-nearest-even conversion (the
reference truncates the fp16 mantissa, src/quantize.rs:633-657).

`QuantizedLinear.forward`: INT8 / Q8_0 weights whose groups are whole rows multiply on the int8
tensor cores with dynamically quantised activations; every other format is dequantised to bf16 by
a kernel and multiplied by the bf16 GEMM (fp32 accumulate), with the bias in the epilogue.
"""
from __future__ import annotations

import enum
from typing import List, Optional

import torch

from . import nn
from .ops import gemm as G
from .ops import quant_kernels as Q


class QuantFormat(enum.Enum):
    FP16 = "FP16"
    BF16 = "BF16"
    INT8 = "INT8"
    INT4 = "INT4"
    NF4 = "NF4"
    NVFP4 = "NVFP4"
    GGUF_Q4 = "GGUF_Q4"
    GGUF_Q4K = "GGUF_Q4K"
    GGUF_Q8 = "GGUF_Q8"

    def bits(self) -> int:
        if self in (QuantFormat.FP16, QuantFormat.BF16):
            return 16
        if self in (QuantFormat.INT8, QuantFormat.GGUF_Q8):
            return 8
        return 4

    def compression_ratio(self) -> float:
        return 32.0 / self.bits()

    def name_str(self) -> str:
        return {QuantFormat.FP16: "FP16", QuantFormat.BF16: "BF16", QuantFormat.INT8: "INT8", QuantFormat.INT4: "INT4",
                QuantFormat.NF4: "NF4 (NormalFloat 4-bit)", QuantFormat.NVFP4: "NVFP4 (NVIDIA FP4 E2M1)",
                QuantFormat.GGUF_Q4: "GGUF Q4_0", QuantFormat.GGUF_Q4K: "GGUF Q4_K", QuantFormat.GGUF_Q8: "GGUF Q8_0"}[self]


_KERNEL_FMT = {QuantFormat.INT8: Q.Q_INT8, QuantFormat.INT4: Q.Q_INT4, QuantFormat.NF4: Q.Q_NF4, QuantFormat.NVFP4: Q.Q_NVFP4,
               QuantFormat.GGUF_Q4: Q.Q_Q4_0, QuantFormat.GGUF_Q4K: Q.Q_Q4_0, QuantFormat.GGUF_Q8: Q.Q_Q8_0}


class QuantizedTensor:
    """`data` uint8 (device), `scales` fp32 (device), `shape`, `group_size` as the reference's fields."""

    def __init__(self, format: QuantFormat, data: torch.Tensor, scales: torch.Tensor, shape, group_size: int):
        self.format, self.data, self.scales, self.shape, self.group_size = format, data, scales, list(shape), group_size

    @staticmethod
    def quantize(tensor: torch.Tensor, format: QuantFormat, group_size: int = 0) -> "QuantizedTensor":
        t = tensor.detach()
        n = t.numel()
        gs = n if group_size == 0 else group_size
        if format in (QuantFormat.FP16, QuantFormat.BF16):
            dt = torch.float16 if format == QuantFormat.FP16 else torch.bfloat16
            data = t.to(dt).contiguous().reshape(-1).view(torch.uint8)
            return QuantizedTensor(format, data, torch.empty(0, dtype=torch.float32, device=t.device), t.shape, 0)
        if format in (QuantFormat.GGUF_Q4, QuantFormat.GGUF_Q4K, QuantFormat.GGUF_Q8):
            gs = min(gs, 32)
        stored = QuantFormat.GGUF_Q4 if format == QuantFormat.GGUF_Q4K else format      # as the reference records it
        data, scales = Q.quant_group(t, max(gs, 1), _KERNEL_FMT[format])
        return QuantizedTensor(stored, data, scales, t.shape, max(gs, 1))

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def dequantize(self, out_dtype=torch.float32) -> torch.Tensor:
        n = self.numel()
        if self.format in (QuantFormat.FP16, QuantFormat.BF16):
            dt = torch.float16 if self.format == QuantFormat.FP16 else torch.bfloat16
            return self.data.view(dt)[:n].to(out_dtype).reshape(self.shape)
        return Q.dequant_group(self.data, self.scales, n, self.group_size, _KERNEL_FMT[self.format], out_dtype).reshape(self.shape)

    def mem_bytes(self) -> int:
        return self.data.numel() + self.scales.numel() * 4

    def compression_ratio(self) -> float:
        return self.numel() * 4 / self.mem_bytes()

    def quantization_error(self, original: torch.Tensor) -> float:
        o = original.detach().float().to(self.data.device)
        return float((o - self.dequantize()).abs().sum() / max(o.numel(), 1))


class QuantizedLinear(nn.Module):
    def __init__(self, weight: QuantizedTensor, bias: Optional[torch.Tensor], in_features: int, out_features: int):
        self.weight, self.bias, self.in_features, self.out_features = weight, bias, in_features, out_features
        self.mx = None          # block-scaled copy of the weight for the tensor-core path (from_linear(tensor_core=True))

    @staticmethod
    def from_linear(layer: nn.Linear, format: QuantFormat, group_size: int = 0, tensor_core: bool = False) -> "QuantizedLinear":
        """`tensor_core=True` (NVFP4 only, in_features a multiple of 256) additionally stores the weight as e2m1 with ue4m3
        block scales, and `forward` on a GPU then multiplies 4-bit operands on the tensor core (ops/mx.py) instead of
        dequantising the weight to bf16."""
        b = layer.bias.detach().float().clone() if layer.bias is not None else None
        q = QuantizedLinear(QuantizedTensor.quantize(layer.weight, format, group_size), b, layer.weight.shape[1], layer.weight.shape[0])
        if tensor_core:
            if format != QuantFormat.NVFP4 or layer.weight.shape[1] % 256 != 0:
                raise ValueError("the tensor-core path takes NVFP4 weights with in_features a multiple of 256")
            from .ops import mx
            q.mx = mx.quantize_mx(layer.weight.detach(), "nvfp4")
        return q

    def _rowwise_int8(self) -> bool:
        w = self.weight
        return w.format in (QuantFormat.INT8, QuantFormat.GGUF_Q8) and w.group_size == self.in_features and len(w.shape) == 2

    def forward(self, x: torch.Tensor, out_dtype=torch.float32, act: str = "none") -> torch.Tensor:
        a = x.detach().reshape(-1, x.shape[-1])
        if self.mx is not None and a.is_cuda:
            from .ops import mx
            y = mx.gemm_mx(mx.quantize_mx(a, "nvfp4"), self.mx, torch.float32)
            if self.bias is not None:
                y = y + self.bias
            y = G.act_ref(y, act).to(out_dtype)
        elif self._rowwise_int8():
            aq, a_scale = Q.quant_rows(a, "int8")
            wq = self.weight.data.view(torch.int8).view(self.out_features, self.in_features)
            y = G.gemm(aq, wq, row_scale=a_scale, col_scale=self.weight.scales, bias=self.bias, act=act, out_dtype=out_dtype)
        elif a.is_cuda:
            w = self.weight.dequantize(torch.bfloat16).reshape(self.out_features, self.in_features)
            y = G.gemm(a.to(torch.bfloat16), w, bias=self.bias, act=act, out_dtype=out_dtype)
        else:
            y = a.float() @ self.weight.dequantize().reshape(self.out_features, self.in_features).t()
            if self.bias is not None:
                y = y + self.bias
            y = G.act_ref(y, act).to(out_dtype)
        return y.reshape(*x.shape[:-1], self.out_features)

    def parameters(self):
        return []


class QuantizedModel:
    """Quantises a model's parameter list pairwise (weight, next tensor as its bias), as
    src/quantize.rs:756-789 does; `forward` chains the layers with ReLU between them when
    `activation="relu"` (the reference exposes only the layer list)."""

    def __init__(self, layers: List[QuantizedLinear], format: QuantFormat):
        self._layers, self.format = layers, format

    @staticmethod
    def from_model(model, format: QuantFormat, group_size: int = 0) -> "QuantizedModel":
        params = list(model.parameters())
        layers, i = [], 0
        while i < len(params):
            w = params[i]
            b = params[i + 1] if i + 1 < len(params) else None
            qt = QuantizedTensor.quantize(w, format, group_size)
            out_f = w.shape[0] if w.dim() >= 1 else 0
            in_f = w.shape[1] if w.dim() >= 2 else 0
            layers.append(QuantizedLinear(qt, b.detach().float().reshape(-1).clone() if b is not None else None, in_f, out_f))
            i += 2 if b is not None else 1
        return QuantizedModel(layers, format)

    def mem_bytes(self) -> int:
        return sum(l.weight.mem_bytes() + (l.bias.numel() * 4 if l.bias is not None else 0) for l in self._layers)

    def compression_ratio(self) -> float:
        total = sum(l.weight.numel() for l in self._layers)
        return total * 4 / max(self.mem_bytes(), 1)

    def layers(self) -> List[QuantizedLinear]:
        return self._layers

    def forward(self, x: torch.Tensor, activation: str = "relu") -> torch.Tensor:
        h = x
        for i, l in enumerate(self._layers):
            h = l.forward(h, act=activation if i + 1 < len(self._layers) else "none")     # ReLU rides the GEMM epilogue
        return h


def quantize(tensor: torch.Tensor, format: QuantFormat, group_size: int = 0) -> QuantizedTensor:
    return QuantizedTensor.quantize(tensor, format, group_size)


# The reference exports both a module and a function called `quantize` from its crate root. Python has
# one namespace, so the module object itself is made callable: `pkg.quantize(t, fmt)` and
# `pkg.quantize.QuantFormat` both work.
import sys as _sys
import types as _types


class _CallableModule(_types.ModuleType):
    def __call__(self, tensor, format, group_size=0):
        return QuantizedTensor.quantize(tensor, format, group_size)


_sys.modules[__name__].__class__ = _CallableModule



from ._compat import install as _install  # noqa: E402

_install(globals())
