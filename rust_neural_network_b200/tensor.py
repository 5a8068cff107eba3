"""`Tensor`: the reference's tensor API (rust-nn src/tensor.rs) as a thin facade over `torch.Tensor`.

The reference implements its own tape (`Op` enum + topological backward, src/tensor.rs:67-130,
1158-2023); here PyTorch's autograd is the tape and each fused op maps to one of this package's
kernels through `ops.functional`. Method names and semantics follow the reference:
`transpose()` reverses ALL axes (src/tensor.rs:1126-1133), `sum()` is a full reduction to a 0-d
tensor, `mean/max/min` return Python floats, `argmax` is a flat index, `clamp/round` record no
gradient, constructors `he` / `xavier` return tensors that require grad.
"""
from __future__ import annotations

import enum
import math
from typing import Optional, Sequence

import torch

from .error import ShapeMismatch
from .ops import functional as F
from .ops import kernels as K


class Device(enum.Enum):
    Cpu = "cpu"
    Gpu = "cuda"
    Cuda = "cuda"
    Metal = "metal"      # accepted for API parity; there is no Metal backend


class FusedAct(enum.Enum):
    Identity = "none"
    Relu = "relu"
    Gelu = "gelu"
    Silu = "silu"
    Sigmoid = "sigmoid"
    Tanh = "tanh"

    def to_u8(self) -> int:
        """Identity 0, Relu 1 as in the reference (src/tensor.rs:134-152); the activations it does not have follow."""
        return list(FusedAct).index(self)

    @staticmethod
    def from_u8(v: int) -> "FusedAct":
        members = list(FusedAct)
        return members[v] if 0 <= v < len(members) else FusedAct.Identity


class KernelKind(enum.IntEnum):
    Elu = 0
    Relu2 = 1

    def to_u8(self) -> int:
        return int(self)

    @staticmethod
    def from_u8(v: int) -> "KernelKind":
        return KernelKind(v)


def _unwrap(x):
    return x.t if isinstance(x, Tensor) else x


class Tensor:
    __slots__ = ("t",)

    def __init__(self, data, requires_grad: bool = False):
        if isinstance(data, Tensor):
            data = data.t
        if not isinstance(data, torch.Tensor):
            data = torch.as_tensor(data, dtype=torch.float32)
        if requires_grad and not data.requires_grad:
            data = data.detach().clone().requires_grad_(True) if not data.is_leaf else data.requires_grad_(True)
        self.t = data

    # ---- constructors
    @staticmethod
    def new(data, requires_grad: bool = False) -> "Tensor":
        return Tensor(torch.as_tensor(data, dtype=torch.float32).clone(), requires_grad)

    @staticmethod
    def zeros(shape: Sequence[int]) -> "Tensor":
        return Tensor(torch.zeros(*shape))

    @staticmethod
    def ones(shape: Sequence[int]) -> "Tensor":
        return Tensor(torch.ones(*shape))

    @staticmethod
    def from_vec(data: Sequence[float], shape: Sequence[int]) -> "Tensor":
        n = 1
        for s in shape:
            n *= int(s)
        if n != len(data):
            raise ShapeMismatch(tuple(shape), (len(data),), "Shape mismatch")
        return Tensor(torch.tensor(list(data), dtype=torch.float32).view(*shape))

    @staticmethod
    def randn(shape: Sequence[int]) -> "Tensor":
        return Tensor(torch.randn(*shape))

    @staticmethod
    def he(shape: Sequence[int]) -> "Tensor":
        return Tensor(torch.randn(*shape) * math.sqrt(2.0 / shape[-1]), requires_grad=True)

    @staticmethod
    def xavier(shape: Sequence[int]) -> "Tensor":
        fan_in, fan_out = shape[-1], shape[0]
        return Tensor(torch.randn(*shape) * math.sqrt(2.0 / (fan_in + fan_out)), requires_grad=True)

    # ---- properties
    def shape(self):
        return list(self.t.shape)

    def ndim(self) -> int:
        return self.t.dim()

    def len(self) -> int:
        return self.t.numel()

    def __len__(self):
        return self.t.numel()

    def is_empty(self) -> bool:
        return self.t.numel() == 0

    def data(self) -> torch.Tensor:
        return self.t.detach()

    def flat_data(self):
        return self.t.detach().float().reshape(-1).cpu().tolist()

    def with_data_slice(self, fn):
        return fn(self.t.detach().reshape(-1))

    def grad(self) -> Optional[torch.Tensor]:
        return self.t.grad

    def requires_grad(self) -> bool:
        return self.t.requires_grad

    def set_requires_grad(self, flag: bool) -> "Tensor":
        self.t.requires_grad_(flag)
        return self

    def clone(self) -> "Tensor":
        """Another handle on the same storage, as cloning the reference's `Arc`-backed tensor gives (src/tensor.rs:34-40)."""
        return Tensor(self.t)

    def zero_grad(self) -> None:
        if self.t.grad is not None:
            self.t.grad.zero_()

    def to_device(self, device) -> "Tensor":
        dev = device.value if isinstance(device, Device) else device
        if dev == "metal":
            raise ValueError("no Metal backend: devices are 'cpu' and 'cuda'")
        rg = self.t.requires_grad
        t = self.t.detach().to(dev)
        return Tensor(t.requires_grad_(rg))

    def device(self) -> Device:
        return Device.Cuda if self.t.is_cuda else Device.Cpu

    # ---- arithmetic (broadcasting; gradients are un-broadcast by autograd)
    def _bin(self, other, op):
        a, b = self.t, _unwrap(other)
        if not isinstance(b, torch.Tensor):
            b = torch.tensor(float(b), dtype=a.dtype, device=a.device)
        if a.is_cuda and a.shape == b.shape and a.dtype == b.dtype and a.dtype in (torch.float32, torch.bfloat16):
            return Tensor(_EwFn.apply(a, b, op))
        return Tensor({"add": torch.add, "sub": torch.sub, "mul": torch.mul}[op](a, b))

    def add(self, o): return self._bin(o, "add")
    def sub(self, o): return self._bin(o, "sub")
    def mul(self, o): return self._bin(o, "mul")
    __add__ = add
    __sub__ = sub
    __mul__ = mul

    def matmul(self, other) -> "Tensor":
        a, b = self.t, _unwrap(other)
        if a.dim() != 2 or b.dim() != 2:
            raise ShapeMismatch((2,), (a.dim(), b.dim()), "matmul supports 2-D x 2-D")
        if a.shape[1] != b.shape[0]:
            raise ShapeMismatch(tuple(a.shape), tuple(b.shape), "matmul inner dimensions")
        return Tensor(F.matmul(a, b))

    def sum(self) -> "Tensor":
        return Tensor(self.t.sum())

    def reshape(self, shape) -> "Tensor":
        return Tensor(self.t.reshape(*shape))

    def transpose(self) -> "Tensor":
        return Tensor(self.t.permute(*reversed(range(self.t.dim()))))

    def permute(self, axes) -> "Tensor":
        return Tensor(self.t.permute(*axes))

    def relu(self): return Tensor(F.relu(self.t))
    def sigmoid(self): return Tensor(F.sigmoid(self.t))
    def silu(self): return Tensor(F.silu(self.t))
    def softplus(self): return Tensor(F.softplus(self.t))
    def tanh(self): return Tensor(F.tanh(self.t))
    def gelu(self): return Tensor(F.gelu(self.t))

    def clamp(self, lo: float, hi: float) -> "Tensor":
        return Tensor(K.unary(self.t.detach(), "clamp", lo, hi))

    def round(self) -> "Tensor":
        return Tensor(K.unary(self.t.detach(), "round"))

    def mean(self) -> float: return float(self.t.detach().float().mean())
    def max(self) -> float: return float(K.reduce_all(self.t.detach(), "max"))
    def min(self) -> float: return float(K.reduce_all(self.t.detach(), "min"))
    def argmax(self) -> int: return int(self.t.detach().reshape(-1).argmax())
    def get_idx(self, i: int) -> float: return float(self.t.detach().reshape(-1)[i])
    def get(self, idx: Sequence[int]) -> float: return float(self.t.detach()[tuple(idx)])

    # ---- fused losses
    def cross_entropy_logits(self, target) -> "Tensor":
        return Tensor(F.cross_entropy(self.t, _unwrap(target)))

    def bce_with_logits(self, target): return Tensor(F.pointwise_loss(self.t, _unwrap(target), "bce_logits"))
    def bce(self, target): return Tensor(F.pointwise_loss(self.t, _unwrap(target), "bce"))
    def l1_loss(self, target): return Tensor(F.pointwise_loss(self.t, _unwrap(target), "l1"))
    def huber_loss(self, target, delta: float = 1.0): return Tensor(F.pointwise_loss(self.t, _unwrap(target), "huber", delta))

    # ---- fused ops (static in the reference)
    @staticmethod
    def flash_attention(q, k, v, scale: float, causal: bool = False) -> "Tensor":
        """[B, S, d] x3 -> [B, S, d] (src/tensor.rs:618)."""
        qt, kt, vt = (_unwrap(x).unsqueeze(2) for x in (q, k, v))
        return Tensor(F.flash_attention(qt, kt, vt, scale, causal).squeeze(2))

    @staticmethod
    def linear_attention(q, k, v, scale: float, eps: float, causal: bool, kind: KernelKind = KernelKind.Elu) -> "Tensor":
        from .ops.linear_attention import linear_attention
        qt, kt, vt = (_unwrap(x).unsqueeze(2) for x in (q, k, v))
        name = "elu" if int(kind) == 0 else "relu2"
        return Tensor(linear_attention(qt, kt, vt, scale=scale, eps=eps, causal=causal, kind=name).squeeze(2))

    @staticmethod
    def linear_layer(x, w, b=None, act: FusedAct = FusedAct.Identity) -> "Tensor":
        return Tensor(F.linear(_unwrap(x), _unwrap(w), _unwrap(b) if b is not None else None, act.value if isinstance(act, FusedAct) else act))

    @staticmethod
    def selective_scan(delta, b_vec, c_vec, u, a) -> "Tensor":
        from .ops.scan import selective_scan
        return Tensor(selective_scan(_unwrap(u), _unwrap(delta), _unwrap(a), _unwrap(b_vec), _unwrap(c_vec)))

    @staticmethod
    def conv1d_causal(inp, weight) -> "Tensor":
        from .ops.scan import causal_conv1d
        return Tensor(causal_conv1d(_unwrap(inp), _unwrap(weight), None, "none"))

    def layer_norm(self, gamma, beta, eps: float = 1e-5) -> "Tensor":
        return Tensor(F.layer_norm(self.t, _unwrap(gamma), _unwrap(beta), eps))

    @staticmethod
    def apply_rope(x, cos, sin, half_dim: int) -> "Tensor":
        from .position import apply_rope
        return Tensor(apply_rope(_unwrap(x), _unwrap(cos), _unwrap(sin), half_dim))

    # ---- autograd
    def backward(self) -> None:
        if self.t.dim() == 0:
            self.t.backward()
        else:
            self.t.backward(torch.ones_like(self.t))

    def backward_with_grad(self, grad) -> None:
        self.t.backward(_unwrap(grad) if isinstance(grad, (Tensor, torch.Tensor)) else torch.as_tensor(grad, dtype=self.t.dtype, device=self.t.device))

    def __repr__(self):
        return f"Tensor(shape={list(self.t.shape)}, requires_grad={self.t.requires_grad}, device={self.t.device})\n{self.t.detach()}"


class _EwFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, op):
        ctx.op = op
        if op == "mul":
            ctx.save_for_backward(a, b)
        return K.binary(a, b, op)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if ctx.op == "add":
            return g, g, None
        if ctx.op == "sub":
            return g, K.unary(g, "scale", -1.0), None
        a, b = ctx.saved_tensors
        return K.binary(g, b, "mul"), K.binary(g, a, "mul"), None
