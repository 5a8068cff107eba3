"""Mamba (S6) models (rust-nn src/mamba.rs): `MambaBlock`, `Mamba`, `HybridMamba`.

`MambaBlock(d_model, d_state, expand, kernel)` follows the reference exactly by default:
separate biased `in_proj_x` / `in_proj_z`, depthwise causal conv (identity-last-tap init, no bias),
SiLU, a FULL d_inner -> d_inner `proj_delta` + softplus, `proj_b` / `proj_c` d_inner -> d_state,
`A[d, n] = -0.5 (n+1)`, gate `y * silu(z)`, `out_proj`; no D skip, no dt_rank, no norm
(src/mamba.rs:52-126). Parameter order (the checkpoint contract, src/mamba.rs:115-125):
in_proj_x, in_proj_z, conv_weight, a, proj_delta, proj_b, proj_c, out_proj.

`standard=True` switches to the parameterisation of the Mamba LM configuration: low-rank
`dt_rank` projection with a dt bias (inverse-softplus init in [1e-3, 1e-1]), `A = -exp(A_log)` with
`A_log = log(1..d_state)`, a D skip, a conv bias, and a pre-norm + residual LM stack (`MambaLM`).

Kernels: conv1d+SiLU, selective scan with the softplus / dt bias / D skip / SiLU gate fused in, and
the tcgen05 GEMM for every projection.
"""
from __future__ import annotations

import math
from typing import List

import torch

from .. import nn
from ..ops import functional as F
from ..ops.scan import causal_conv1d, selective_scan
from ..ops.transformer import lm_head_ce
from ..parallel.ddp import mark
from .looped_transformer import _add


class MambaBlock(nn.Module):
    def __init__(self, d_model: int, d_state: int, expand: int, kernel_size: int, standard: bool = False,
                 dt_rank: int = 0, init=nn.he_normal):
        self.d_model, self.d_state, self.kernel_size = d_model, d_state, kernel_size
        self.d_inner = expand * d_model
        self.standard = standard
        di = self.d_inner
        self.in_proj_x = nn.Linear(d_model, di, init=init)
        self.in_proj_z = nn.Linear(d_model, di, init=init)
        conv = torch.zeros(di, kernel_size)
        if standard:
            conv = (torch.rand(di, kernel_size) * 2 - 1) / math.sqrt(kernel_size)
        else:
            conv[:, kernel_size - 1] = 1.0
        self.conv_weight = nn._param(conv)
        if standard:
            self.dt_rank = dt_rank or math.ceil(d_model / 16)
            self.a = nn._param(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32)).repeat(di, 1))   # A_log
            self.proj_delta = nn.Linear(di, self.dt_rank, bias=False, init=init)       # x -> dt_rank
            self.dt_up = nn.Linear(self.dt_rank, di, bias=False, init=lambda s, generator=None: (torch.rand(*s) * 2 - 1) * self.dt_rank ** -0.5)
            dt = torch.exp(torch.rand(di) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp_min(1e-4)
            self.dt_bias = nn._param(dt + torch.log(-torch.expm1(-dt)))                   # inverse softplus
            self.d_skip = nn._param(torch.ones(di))
            self.conv_bias = nn._param(torch.zeros(di))
        else:
            self.dt_rank = 0
            self.a = nn._param((-(torch.arange(d_state, dtype=torch.float32) + 1) * 0.5).repeat(di, 1))
            self.proj_delta = nn.Linear(di, di, init=init)
        self.proj_b = nn.Linear(di, d_state, init=init)
        self.proj_c = nn.Linear(di, d_state, init=init)
        self.out_proj = nn.Linear(di, d_model, init=init)

    def forward(self, x):
        xs = self.in_proj_x(x)                                         # [B, S, d_inner]
        z = self.in_proj_z(x)
        if self.standard:
            xa = causal_conv1d(xs, self.conv_weight, self.conv_bias, "silu")
            dt = self.dt_up(self.proj_delta(xa))
            b_vec, c_vec = self.proj_b(xa), self.proj_c(xa)
            A = -torch.exp(self.a.float())
            y = selective_scan(xa, dt, A, b_vec, c_vec, self.d_skip, z, self.dt_bias, True)
        else:
            xa = causal_conv1d(xs, self.conv_weight, None, "silu")
            delta = self.proj_delta(xa)                                # softplus is applied inside the scan kernel
            b_vec, c_vec = self.proj_b(xa), self.proj_c(xa)
            y = selective_scan(xa, delta, self.a, b_vec, c_vec, None, z, None, True)
        return self.out_proj(y)

    def parameters(self):
        p = self.in_proj_x.parameters() + self.in_proj_z.parameters() + [self.conv_weight, self.a] + self.proj_delta.parameters()
        p += self.proj_b.parameters() + self.proj_c.parameters() + self.out_proj.parameters()
        if self.standard:
            p += self.dt_up.parameters() + [self.dt_bias, self.d_skip, self.conv_bias]
        return p


class Mamba(nn.Module):
    """Stack of blocks with `x = x + block(x)` (src/mamba.rs:131-171)."""

    def __init__(self, d_model: int, d_state: int, expand: int, kernel_size: int, num_layers: int, **kw):
        self.blocks = [MambaBlock(d_model, d_state, expand, kernel_size, **kw) for _ in range(num_layers)]

    def children(self):
        return list(self.blocks)

    def forward(self, x):
        for b in self.blocks:
            x = _add(x, b(x))
        return x

    def parameters(self):
        ps = []
        for b in self.blocks:
            ps += b.parameters()
        return ps


class HybridMamba(nn.Module):
    """User-ordered list of blocks, each applied residually (src/mamba.rs:179-233)."""

    def __init__(self, d_model: int):
        self.d_model = d_model
        self.blocks: List[nn.Module] = []

    def with_block(self, block):
        self.blocks.append(block); return self

    def with_mamba(self, d_state: int, expand: int, kernel_size: int):
        self.blocks.append(MambaBlock(self.d_model, d_state, expand, kernel_size)); return self

    def with_layer(self, layer):
        self.blocks.append(layer); return self

    def children(self):
        return list(self.blocks)

    def forward(self, x):
        for b in self.blocks:
            x = _add(x, b(x))
        return x

    def parameters(self):
        ps = []
        for b in self.blocks:
            ps += b.parameters()
        return ps


class MambaLM(nn.Module):
    """Token embedding -> num_layers x (LayerNorm -> MambaBlock(standard) -> residual) -> LayerNorm -> LM head."""

    def __init__(self, vocab: int, d_model: int, num_layers: int, d_state: int = 16, d_conv: int = 4, expand: int = 2,
                 dt_rank: int = 0, init_std: float = 0.02):
        init = nn.normal_init(init_std)
        self.tok = nn.Embedding(vocab, d_model, std=init_std)
        self.norms = [nn.LayerNorm(d_model) for _ in range(num_layers)]
        self.blocks = [MambaBlock(d_model, d_state, expand, d_conv, standard=True, dt_rank=dt_rank, init=init) for _ in range(num_layers)]
        self.ln_final = nn.LayerNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab, bias=False, init=init)

    def children(self):
        return [self.tok] + self.norms + self.blocks + [self.ln_final, self.lm_head]

    def hidden(self, ids):
        h = self.tok(ids)
        for i, (n, b) in enumerate(zip(self.norms, self.blocks)):
            h = mark(h, i + 1)
            h = _add(h, b(n(h)))
        return self.ln_final(mark(h, len(self.blocks) + 1))

    def dp_groups(self):
        """Parameter groups in forward order; `mark(h, k)` sits in front of group k."""
        return ([self.tok.parameters()] + [n.parameters() + b.parameters() for n, b in zip(self.norms, self.blocks)]
                + [self.ln_final.parameters() + self.lm_head.parameters()])

    def forward(self, ids):
        return self.lm_head(self.hidden(ids))

    def loss(self, ids, labels):
        return lm_head_ce(self.hidden(ids), self.lm_head.weight, None, labels)

    def parameters(self):
        ps = self.tok.parameters()
        for n, b in zip(self.norms, self.blocks):
            ps += n.parameters() + b.parameters()
        return ps + self.ln_final.parameters() + self.lm_head.parameters()
