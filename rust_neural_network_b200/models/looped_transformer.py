"""Transformer family (rust-nn src/looped_transformer.rs): `MultiHeadAttention`, `TransformerBlock`,
`LoopedTransformer` (one shared block applied `num_loops` times with a per-loop time embedding and
optional ACT halting) and the plain `Transformer` stack.

Structure and parameter order follow the reference; options the BASELINE configs need are added as
keyword arguments with reference-compatible defaults: `causal` (reference: non-causal),
`layers_per_block` (reference: one shared `TransformerBlock`), bf16 compute via `to_device`.
On CUDA with bf16 activations a block runs as ONE hand-written fused function
(`ops/transformer.py`); otherwise it is composed from the differentiable per-op kernels.
"""
from __future__ import annotations

import enum
import math
from typing import List

import torch

from .. import nn
from ..ops import functional as F
from ..ops import kernels as K
from ..ops.transformer import transformer_block


class AttentionKind(enum.Enum):
    Flash = 0     # exact softmax attention (default), src/looped_transformer.rs:32-39
    Linear = 1    # ELU+1 linear attention


def sinusoidal_embedding(t: float, dim: int, device=None) -> torch.Tensor:
    """[1, dim] embedding with interleaved sin/cos, max_period 1e4 (rust-nn src/diffusion.rs:89-105)."""
    half = dim // 2
    i = torch.arange(half, dtype=torch.float32, device=device)
    freq = torch.exp(-math.log(10000.0) * i / max(half, 1))
    ang = float(t) * freq
    out = torch.zeros(1, dim, dtype=torch.float32, device=device)
    out[0, 0:2 * half:2] = torch.sin(ang)
    out[0, 1:2 * half:2] = torch.cos(ang)
    return out


class MultiHeadAttention(nn.Module):
    """Four biased Linears (q, k, v, out); heads split as strided views of the projections (no
    permute copies); Flash (softmax) or Linear (ELU+1) attention (src/looped_transformer.rs:59-143).
    The q/k/v weights are tagged as one fusion group so an optimizer lays them out as a contiguous
    [3d, d] matrix and the block kernel runs a single QKV GEMM."""

    def __init__(self, d_model: int, heads: int, causal: bool = False, init=nn.he_normal):
        assert d_model % heads == 0
        self.d_model, self.heads, self.causal = d_model, heads, causal
        self.kind = AttentionKind.Flash
        self.q_proj = nn.Linear(d_model, d_model, init=init)
        self.k_proj = nn.Linear(d_model, d_model, init=init)
        self.v_proj = nn.Linear(d_model, d_model, init=init)
        self.out_proj = nn.Linear(d_model, d_model, init=init)
        gw, gb = object(), object()
        for i, lin in enumerate((self.q_proj, self.k_proj, self.v_proj)):
            lin.weight._fuse_group, lin.weight._fuse_index = gw, i
            lin.bias._fuse_group, lin.bias._fuse_index = gb, i

    def with_attention(self, kind: AttentionKind):
        self.kind = kind
        return self

    def forward(self, x, residual=None):
        B, S, d = x.shape
        H, hd = self.heads, d // self.heads
        q = self.q_proj(x).view(B, S, H, hd)
        k = self.k_proj(x).view(B, S, H, hd)
        v = self.v_proj(x).view(B, S, H, hd)
        if self.kind == AttentionKind.Flash:
            o = F.flash_attention(q, k, v, 1.0 / math.sqrt(hd), self.causal)
        else:
            from ..ops.linear_attention import linear_attention
            o = linear_attention(q, k, v, scale=1.0, eps=1e-6, causal=self.causal, kind="elu")
        return self.out_proj(o.reshape(B, S, d), residual=residual)

    def parameters(self):
        return self.q_proj.parameters() + self.k_proj.parameters() + self.v_proj.parameters() + self.out_proj.parameters()


class TransformerBlock(nn.Module):
    """Pre-norm block: h = x + attn(LN1 x); out = h + FF(LN2 h), FF = Linear -> GELU -> Linear
    (src/looped_transformer.rs:150-202). Parameter order: ln1, attn, ln2, ff."""

    def __init__(self, d_model: int, heads: int, ff_dim: int, causal: bool = False, init=nn.he_normal):
        self.ln1 = nn.LayerNorm(d_model)
        self.attn = MultiHeadAttention(d_model, heads, causal, init=init)
        self.ln2 = nn.LayerNorm(d_model)
        self.ff1 = nn.Linear(d_model, ff_dim, init=init)
        self.ff2 = nn.Linear(ff_dim, d_model, init=init)
        self.causal = causal

    def with_attention(self, kind: AttentionKind):
        self.attn.with_attention(kind)
        return self

    def forward(self, x):
        fused = (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and self.attn.kind == AttentionKind.Flash
                 and (x.shape[-1] // self.attn.heads) in (64, 128))
        if fused:
            return transformer_block(x, self, self.causal)
        h = self.attn(self.ln1(x), residual=x)
        a = F.linear(self.ln2(h), self.ff1.weight, self.ff1.bias, "gelu", None)
        return self.ff2(a, residual=h)

    def parameters(self):
        return self.ln1.parameters() + self.attn.parameters() + self.ln2.parameters() + self.ff1.parameters() + self.ff2.parameters()


class _BlockStack(nn.Module):
    def __init__(self, blocks: List[TransformerBlock]):
        self.blocks = blocks

    def children(self):
        return list(self.blocks)

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return x

    def parameters(self):
        ps = []
        for b in self.blocks:
            ps.extend(b.parameters())
        return ps


class LoopedTransformer(nn.Module):
    """embed (Linear) -> per loop t: cond = h + time_proj(sinusoid(t)); h = cond + block(cond) -> LN -> head
    (src/looped_transformer.rs:251-358; the block is itself residual, so the residual is applied twice,
    as in the reference). Parameter order: embed, block, ln_final, head, time_proj, [halt_unit].
    ACT halting: accumulate sigmoid(halt_unit(h)) of the first element and stop once it reaches the
    threshold (default 0.9); the accumulator is read back once per loop, as in the reference."""

    def __init__(self, input_dim: int, d_model: int, heads: int, ff_dim: int, output_dim: int, num_loops: int,
                 causal: bool = False, layers_per_block: int = 1, init=nn.he_normal):
        self.d_model, self.num_loops = d_model, num_loops
        self.embed = nn.Linear(input_dim, d_model, init=init)
        self.block = _BlockStack([TransformerBlock(d_model, heads, ff_dim, causal, init=init) for _ in range(layers_per_block)])
        self.ln_final = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, output_dim, init=init)
        self.time_proj = nn.Sequential(nn.Linear(d_model, d_model, init=init), nn.GELU(), nn.Linear(d_model, d_model, init=init))
        self.halt_unit = None
        self.halt_threshold = 0.9
        self.adaptive = False

    def with_adaptive_halting(self, threshold: float = 0.9):
        self.adaptive = True
        self.halt_threshold = threshold
        if self.halt_unit is None:
            self.halt_unit = nn.Linear(self.d_model, 1)
            self.halt_unit.to_device(self.embed.weight.device)
        return self

    def with_attention(self, kind: AttentionKind):
        for b in self.block.blocks:
            b.with_attention(kind)
        return self

    def time_conditioning(self, device, dtype) -> torch.Tensor:
        """[num_loops, d] time embeddings through time_proj (one pair of small GEMMs per step)."""
        cache = getattr(self, "_time_emb", None)
        if cache is None or cache.device != device or cache.dtype != dtype or cache.shape[0] != self.num_loops:
            emb = torch.cat([sinusoidal_embedding(t, self.d_model) for t in range(self.num_loops)], 0)
            cache = emb.to(device=device, dtype=dtype)
            self._time_emb = cache          # constant table: built once, not per step
        return self.time_proj(cache)

    def trunk(self, h):
        """Apply the looped block to already-embedded activations; returns (h, loops_run)."""
        tc = self.time_conditioning(h.device, h.dtype)
        loops = 0
        halt_acc = 0.0
        for t in range(self.num_loops):
            cond = _add_row(h, tc[t])
            h = _add(cond, self.block(cond))
            loops += 1
            if self.adaptive:
                hv = torch.sigmoid(self.halt_unit(h).float()).reshape(-1)[0]
                halt_acc += float(hv)
                if halt_acc >= self.halt_threshold:
                    break
        return h, loops

    def forward_with_loops(self, x):
        h = self.embed(x)
        h, loops = self.trunk(h)
        return self.head(self.ln_final(h)), loops

    def forward(self, x):
        return self.forward_with_loops(x)[0]

    def parameters(self):
        ps = (self.embed.parameters() + self.block.parameters() + self.ln_final.parameters() + self.head.parameters()
              + self.time_proj.parameters())
        if self.adaptive and self.halt_unit is not None:
            ps += self.halt_unit.parameters()
        return ps


class Transformer(nn.Module):
    """Non-looped stack of blocks (src/looped_transformer.rs:365-436). Parameter order: embed, blocks,
    ln_final, head. `with_attention` re-initialises all blocks, as the reference does."""

    def __init__(self, input_dim: int, d_model: int, heads: int, ff_dim: int, output_dim: int, num_layers: int,
                 causal: bool = False, init=nn.he_normal):
        self._cfg = (d_model, heads, ff_dim, num_layers, causal, init)
        self.embed = nn.Linear(input_dim, d_model, init=init)
        self.blocks = [TransformerBlock(d_model, heads, ff_dim, causal, init=init) for _ in range(num_layers)]
        self.ln_final = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, output_dim, init=init)

    def with_attention(self, kind: AttentionKind):
        d_model, heads, ff_dim, num_layers, causal, init = self._cfg
        dev = self.embed.weight.device
        self.blocks = [TransformerBlock(d_model, heads, ff_dim, causal, init=init).with_attention(kind) for _ in range(num_layers)]
        for b in self.blocks:
            b.to_device(dev, self.compute_dtype)
        return self

    def forward(self, x):
        h = self.embed(x)
        for b in self.blocks:
            h = b(h)
        return self.head(self.ln_final(h))

    def parameters(self):
        ps = self.embed.parameters()
        for b in self.blocks:
            ps += b.parameters()
        return ps + self.ln_final.parameters() + self.head.parameters()


# ----------------------------------------------------------------------------- small differentiable helpers
class _AddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        return K.binary(a, b, "add")

    @staticmethod
    def backward(ctx, g):
        return g, g


class _AddRowFn(torch.autograd.Function):
    """a [.., d] + row [d] (broadcast), gradient of the row is the column sum."""

    @staticmethod
    def forward(ctx, a, row):
        ctx.row_dtype = row.dtype
        return K.binary(a, row.to(a.dtype), "add")

    @staticmethod
    def backward(ctx, g):
        d = g.shape[-1]
        return g, K.colsum(g.reshape(-1, d)).to(ctx.row_dtype)


def _add(a, b):
    return _AddFn.apply(a, b)


def _add_row(a, row):
    return _AddRowFn.apply(a, row)


from .._compat import accept_wrapped as _accept_wrapped  # noqa: E402

LoopedTransformer.forward_with_loops = _accept_wrapped(LoopedTransformer.forward_with_loops)   # (output, loops used) for a wrapped input too

from .._compat import alias_fields as _alias_fields  # noqa: E402

# src/looped_transformer.rs:60-70, 150-157, 380-388
_alias_fields(MultiHeadAttention, num_heads="heads", head_dim=lambda self: self.d_model // self.heads, attention="kind")
_alias_fields(TransformerBlock, d_model=lambda self: self.attn.d_model, ff_dim=lambda self: self.ff1.weight.shape[0],
              ff=lambda self: nn.Sequential(self.ff1, nn.GELU(), self.ff2))
_alias_fields(Transformer, d_model=lambda self: self.blocks[0].attn.d_model, num_heads=lambda self: self.blocks[0].attn.heads,
              ff_dim=lambda self: self.blocks[0].ff1.weight.shape[0])
