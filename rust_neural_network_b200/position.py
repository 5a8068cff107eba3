"""Positional encodings (rust-nn src/position.rs): RoPE (+ YaRN), CARoPE, ALiBi, sinusoidal and
learned additive encodings.

RoPE uses the rotate-half convention with duplicated-half `[seq, dim]` cos/sin tables, base 10000;
YaRN scales the base by `scale^(d/(d-2))` (src/position.rs:34-72). The rotation is the `b200_rope`
CUDA kernel with an exact backward (the inverse rotation).
"""
from __future__ import annotations

import enum
import math
from typing import List

import torch

from . import _native as nv
from . import nn

nv.register_sigs({"b200_rope": [nv.c_void_p, nv.c_void_p, nv.c_void_p, nv.c_void_p, nv.c_ll, nv.c_int, nv.c_int, nv.c_float, nv.c_int, nv.c_void_p]})


def inv_freq(head_dim: int, base: float) -> torch.Tensor:
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    return torch.pow(torch.tensor(float(base)), -(2.0 * i) / head_dim)


def inv_freq_yarn(head_dim: int, base: float, scale: float) -> torch.Tensor:
    return inv_freq(head_dim, base * scale ** (head_dim / (head_dim - 2)))


def build_tables(inv_f: torch.Tensor, seq_len: int):
    pos = torch.arange(seq_len, dtype=torch.float32)[:, None]
    ang = pos * inv_f[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    return torch.cat([cos, cos], 1).contiguous(), torch.cat([sin, sin], 1).contiguous()


def _rope_apply(x, cos, sin, sign: float):
    dim = x.shape[-1]
    seq = x.shape[-2] if x.dim() >= 2 else 1
    half = dim // 2
    if not x.is_cuda:
        c, s = cos[:seq].to(x.device), sin[:seq].to(x.device) * sign
        xf = x.float()
        x1, x2 = xf[..., :half], xf[..., half:]
        return torch.cat([x1 * c[:, :half] - x2 * s[:, :half], x2 * c[:, half:] + x1 * s[:, half:]], -1).to(x.dtype)
    xc = x.contiguous()
    y = torch.empty_like(xc)
    c = cos[:seq].to(x.device, torch.float32).contiguous()
    s = sin[:seq].to(x.device, torch.float32).contiguous()
    leading = xc.numel() // (seq * dim)
    nv.check(nv.cuda().b200_rope(xc.data_ptr(), c.data_ptr(), s.data_ptr(), y.data_ptr(), leading, seq, dim, float(sign),
                                 1 if x.dtype == torch.bfloat16 else 0, nv.stream_ptr()), "rope")
    nv.count_launch()
    return y


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _rope_apply(x, cos, sin, 1.0)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        return _rope_apply(g, cos, sin, -1.0), None, None


def apply_rope(x, cos, sin, half_dim: int):
    """x [..., seq, dim] with dim = 2*half_dim; cos/sin tables [seq, dim] (src/tensor.rs:1077-1124)."""
    dim = x.shape[-1]
    if dim != 2 * half_dim:
        raise ValueError("apply_rope: dim must be 2*half_dim")
    cos = torch.as_tensor(cos, dtype=torch.float32).reshape(-1, dim)
    sin = torch.as_tensor(sin, dtype=torch.float32).reshape(-1, dim)
    seq = x.shape[-2] if x.dim() >= 2 else 1
    if cos.shape[0] < seq:
        raise ValueError("apply_rope: cos/sin table shorter than the sequence")
    return _RopeFn.apply(x, cos, sin)


class RoPE:
    def __init__(self, head_dim: int, max_seq_len: int, base: float = 10000.0, _inv=None):
        self.head_dim, self.max_seq_len, self.base = head_dim, max_seq_len, base
        self.inv_freq = inv_freq(head_dim, base) if _inv is None else _inv
        self.cos, self.sin = build_tables(self.inv_freq, max_seq_len)

    @staticmethod
    def new(head_dim: int, max_seq_len: int) -> "RoPE":
        return RoPE(head_dim, max_seq_len)

    @staticmethod
    def with_base(head_dim: int, max_seq_len: int, base: float) -> "RoPE":
        return RoPE(head_dim, max_seq_len, base)

    @staticmethod
    def yarn(head_dim: int, max_seq_len: int, base: float, scale: float) -> "RoPE":
        r = RoPE(head_dim, max_seq_len, base, _inv=inv_freq_yarn(head_dim, base, scale))
        r._yarn_scale = float(scale)
        return r

    def apply(self, x):
        if x.shape[-1] != self.head_dim:
            raise ValueError(f"RoPE: last dim {x.shape[-1]} must equal head_dim {self.head_dim}")
        seq = x.shape[-2] if x.dim() >= 2 else 1
        if seq > self.max_seq_len:
            raise ValueError(f"RoPE: seq len {seq} exceeds max_seq_len {self.max_seq_len}; extend() or use YaRN scaling")
        return apply_rope(x, self.cos[:seq], self.sin[:seq], self.head_dim // 2)

    def extend(self, new_max: int) -> None:
        if new_max > self.max_seq_len:
            self.max_seq_len = new_max
            self.cos, self.sin = build_tables(self.inv_freq, new_max)


class CARoPE:
    """Context-aware RoPE: per-position phase offsets tanh(emb @ freq_proj) * spread modulate the
    frequencies; the offsets are detached, as in the reference (src/position.rs:229-289)."""

    def __init__(self, head_dim: int, input_dim: int, max_seq_len: int):
        self.head_dim, self.input_dim, self.max_seq_len = head_dim, input_dim, max_seq_len
        self.spread = 0.1
        self.base_inv_freq = inv_freq(head_dim, 10000.0)
        self.freq_proj = torch.nn.Parameter(torch.randn(input_dim, head_dim // 2) * 0.02)

    def with_spread(self, spread: float) -> "CARoPE":
        self.spread = spread
        return self

    def apply(self, x, embeddings):
        seq = x.shape[-2] if x.dim() >= 2 else 1
        if x.shape[-1] != self.head_dim:
            raise ValueError("CARoPE: last dim must equal head_dim")
        if seq > self.max_seq_len:
            raise ValueError(f"CARoPE: seq {seq} exceeds max {self.max_seq_len}")
        half = self.head_dim // 2
        emb = embeddings.detach().float().reshape(-1, embeddings.shape[-1])
        emb_seq = embeddings.shape[-2] if embeddings.dim() >= 2 else 1
        offsets = torch.zeros(seq, half)
        n = min(seq, emb_seq)
        k = min(emb.shape[1], self.input_dim)
        offsets[:n] = (torch.tanh(emb[:n, :k].cpu() @ self.freq_proj.detach().float().cpu()[:k]) * self.spread)
        pos = torch.arange(seq, dtype=torch.float32)[:, None]
        ang = pos * (self.base_inv_freq[None, :] + offsets)
        cos, sin = torch.cos(ang), torch.sin(ang)
        return apply_rope(x, torch.cat([cos, cos], 1), torch.cat([sin, sin], 1), half)

    def parameters(self) -> List[torch.Tensor]:
        return [self.freq_proj]


def alibi_slopes(n: int) -> List[float]:
    return [2.0 ** (-8.0 * h / n) for h in range(1, n + 1)]


class AlibiBias:
    def __init__(self, num_heads: int):
        self.num_heads = num_heads
        self.slopes = alibi_slopes(num_heads)

    def bias_matrix(self, seq_len: int, device="cpu") -> torch.Tensor:
        """[H, S, S] additive (negative) bias: -slope_h * |i - j| (src/position.rs:323-336)."""
        i = torch.arange(seq_len, dtype=torch.float32, device=device)
        dist = (i[:, None] - i[None, :]).abs()
        return -torch.tensor(self.slopes, dtype=torch.float32, device=device)[:, None, None] * dist

    def slope(self, head: int) -> float:
        return self.slopes[head] if 0 <= head < len(self.slopes) else 0.0


class SinusoidalPE:
    """Interleaved [sin, cos, ...] table added to [batch, seq, dim] inputs (src/position.rs:357-415)."""

    def __init__(self, dim: int, max_seq_len: int):
        self.dim, self.max_seq_len = dim, max_seq_len
        half = dim // 2
        pos = torch.arange(max_seq_len, dtype=torch.float32)[:, None]
        j = torch.arange(half, dtype=torch.float32)[None, :]
        ang = pos / torch.pow(torch.tensor(10000.0), 2.0 * j / dim)
        tab = torch.zeros(max_seq_len, dim)
        tab[:, 0:2 * half:2] = torch.sin(ang)
        tab[:, 1:2 * half:2] = torch.cos(ang)
        if dim % 2 == 1:
            tab[:, dim - 1] = torch.sin(pos[:, 0] / (10000.0 ** (2.0 * half / dim)))
        self._table = tab

    def table(self) -> torch.Tensor:
        return self._table

    def apply(self, x):
        seq = x.shape[-2]
        if seq > self.max_seq_len:
            raise ValueError("SinusoidalPE: sequence longer than the table")
        return x + self._table[:seq].to(x.device, x.dtype)


class LearnedPE:
    def __init__(self, dim: int, max_seq_len: int):
        self.dim, self.max_seq_len = dim, max_seq_len
        self.table = torch.nn.Parameter(torch.randn(max_seq_len, dim) * 0.02)

    def init_sinusoidal(self) -> "LearnedPE":
        with torch.no_grad():
            self.table.copy_(SinusoidalPE(self.dim, self.max_seq_len).table())
        return self

    def apply(self, x):
        seq = x.shape[-2]
        if seq > self.max_seq_len:
            raise ValueError("LearnedPE: sequence longer than the table")
        return x + self.table[:seq].to(x.dtype)

    def parameters(self) -> List[torch.Tensor]:
        return [self.table]


class PositionalEncoding:
    """`None | Sinusoidal | Learned` (src/position.rs:486-500)."""

    def __init__(self, kind: str = "none", dim: int = 0, max_seq_len: int = 0):
        self.kind = kind
        self.impl = {"none": None, "sinusoidal": SinusoidalPE, "learned": LearnedPE}[kind]
        if self.impl is not None:
            self.impl = self.impl(dim, max_seq_len)

    @staticmethod
    def none(): return PositionalEncoding("none")
    @staticmethod
    def sinusoidal(dim, max_seq_len): return PositionalEncoding("sinusoidal", dim, max_seq_len)
    @staticmethod
    def learned(dim, max_seq_len): return PositionalEncoding("learned", dim, max_seq_len)

    def apply(self, x):
        return x if self.impl is None else self.impl.apply(x)

    def parameters(self):
        return self.impl.parameters() if isinstance(self.impl, LearnedPE) else []


from ._compat import install as _install  # noqa: E402

_install(globals())

from ._compat import alias_fields as _alias_fields  # noqa: E402

# src/position.rs:82-90, 184-195: `scale` is the YaRN factor the tables were built with (1.0 without YaRN), `base` the rotary base
_alias_fields(RoPE, scale=lambda self: getattr(self, "_yarn_scale", 1.0))
_alias_fields(CARoPE, base=lambda self: 10000.0)
