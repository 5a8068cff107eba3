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

Tensor parallelism (`tp=TPContext`, standard form only): the d_inner channels are sharded over the ranks and the
activations between blocks are sharded over rows (sequence parallel). `in_proj` (x and z halves in one weight) is an
all-gather -> GEMM, conv / scan / gate run on the local channels with no communication, the narrow x-projection
(dt_rank + 2 d_state columns) is a row-parallel GEMM + small all-reduce, `out_proj` is a GEMM -> reduce-scatter with the
residual added in the same kernel (parallel/tp.py). The standard form has no biases on its projections.

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
                 dt_rank: int = 0, init=nn.he_normal, tp=None, generator=None):
        self.d_model, self.d_state, self.kernel_size = d_model, d_state, kernel_size
        self.d_inner = expand * d_model
        self.standard = standard
        self.tp = tp
        self.recompute_scan = False      # True: the scan's state checkpoints are rebuilt in the backward instead of kept
        di = self.d_inner
        if tp is not None:
            if not standard:
                raise ValueError("tensor parallelism is implemented for the standard parameterisation")
            self._init_tp(init, dt_rank, generator)
            return
        bias = not standard
        self.in_proj_x = nn.Linear(d_model, di, bias=bias, init=init)
        self.in_proj_z = nn.Linear(d_model, di, bias=bias, init=init)
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
        self.proj_b = nn.Linear(di, d_state, bias=bias, init=init)
        self.proj_c = nn.Linear(di, d_state, bias=bias, init=init)
        self.out_proj = nn.Linear(di, d_model, bias=bias, init=init)

    # ---------------------------------------------------------------- tensor-parallel form
    def _init_tp(self, init, dt_rank, generator):
        """Every rank draws the FULL tensors from `generator` (same seed everywhere) and keeps its channel slice, so a
        tensor-parallel model starts from the same weights for any world size."""
        tp, d_model, di, N, Kc = self.tp, self.d_model, self.d_inner, self.d_state, self.kernel_size
        if di % tp.world:
            raise ValueError("d_inner must divide by the tensor-parallel world size")
        dl = di // tp.world
        lo, hi = tp.rank * dl, (tp.rank + 1) * dl
        g = generator
        self.dt_rank = dt_rank or math.ceil(d_model / 16)
        R = self.dt_rank
        wx, wz = init((di, d_model), generator=g), init((di, d_model), generator=g)
        self.in_proj = nn._param(torch.cat([wx[lo:hi], wz[lo:hi]], 0))                                   # [2 dl, d_model]
        self.conv_weight = nn._param(((torch.rand(di, Kc, generator=g) * 2 - 1) / math.sqrt(Kc))[lo:hi])
        self.a = nn._param(torch.log(torch.arange(1, N + 1, dtype=torch.float32)).repeat(dl, 1))        # A_log
        wd, wb, wc = init((R, di), generator=g), init((N, di), generator=g), init((N, di), generator=g)
        self.x_proj = nn._param(torch.cat([wd, wb, wc], 0)[:, lo:hi].contiguous())                       # [R + 2N, dl]
        self.dt_up = nn._param((((torch.rand(di, R, generator=g) * 2 - 1) * R ** -0.5))[lo:hi])          # [dl, R]
        dt = torch.exp(torch.rand(di, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp_min(1e-4)
        self.dt_bias = nn._param((dt + torch.log(-torch.expm1(-dt)))[lo:hi])
        self.d_skip = nn._param(torch.ones(dl))
        self.conv_bias = nn._param(torch.zeros(dl))
        self.out_proj = nn._param(init((d_model, di), generator=g)[:, lo:hi].contiguous())               # [d_model, dl]
        for p in self.parameters():
            p._tp_sharded = True

    def forward_tp(self, x_s, seq_len: int, residual=None):
        """x_s [rows_local, d_model] (this rank's rows of the normalised input) -> this rank's rows of
        residual + block(x). The rows of all ranks, in rank order, form a [batch, seq_len] grid."""
        from ..parallel import tp as TP
        tp, dl, N, R = self.tp, self.d_inner // self.tp.world, self.d_state, self.dt_rank
        xz = TP.column_parallel(x_s, self.in_proj, None, tp)                        # [M, 2 dl]
        M = xz.shape[0]
        Bt = M // seq_len
        xs, z = TP.split_cols(xz, dl)
        xs, z = xs.view(Bt, seq_len, dl), z.view(Bt, seq_len, dl)
        xa = causal_conv1d(xs, self.conv_weight, self.conv_bias, "silu")            # [Bt, S, dl]
        xp = TP.row_parallel_all_reduce(xa.reshape(M, dl), self.x_proj, tp)             # [M, R + 2N] identical on all ranks
        dt = F.linear(xp[:, :R], self.dt_up, None, "none", None)                     # [M, dl]
        b_vec, c_vec = xp[:, R:R + N].view(Bt, seq_len, N), xp[:, R + N:].view(Bt, seq_len, N)
        A = -torch.exp(self.a.float())
        y = selective_scan(xa, dt.reshape(Bt, seq_len, dl), A, b_vec, c_vec, self.d_skip, z, self.dt_bias, True, self.recompute_scan)
        return TP.row_parallel(y.reshape(M, dl), self.out_proj, None, residual, tp)  # [rows_local, d_model]

    def forward(self, x):
        if self.tp is not None:
            raise RuntimeError("a tensor-parallel block runs on row-sharded activations: call forward_tp")
        xs = self.in_proj_x(x)                                         # [B, S, d_inner]
        z = self.in_proj_z(x)
        if self.standard:
            xa = causal_conv1d(xs, self.conv_weight, self.conv_bias, "silu")
            # the three bias-free projections of xa as ONE product with their stacked weights: xa ([B*S, d_inner], the
            # widest activation of the block) is read once instead of three times, and its gradient arrives as one
            # matrix instead of three that autograd would have to add
            from ..parallel.tp import split_cols
            R, N = self.dt_rank, self.d_state
            Bt, S = xa.shape[0], xa.shape[1]
            w_cat = torch.cat([self.proj_delta.weight, self.proj_b.weight, self.proj_c.weight], 0)     # [R + 2N, d_inner]
            xp = F.linear(xa.reshape(Bt * S, self.d_inner), w_cat, None, "none", None)
            dlow, bc = split_cols(xp, R)
            b2, c2 = split_cols(bc, N)
            dt = self.dt_up(dlow).view(Bt, S, self.d_inner)
            b_vec, c_vec = b2.view(Bt, S, N), c2.view(Bt, S, N)
            A = -torch.exp(self.a.float())
            y = selective_scan(xa, dt, A, b_vec, c_vec, self.d_skip, z, self.dt_bias, True, self.recompute_scan)
        else:
            xa = causal_conv1d(xs, self.conv_weight, None, "silu")
            delta = self.proj_delta(xa)                                # softplus is applied inside the scan kernel
            b_vec, c_vec = self.proj_b(xa), self.proj_c(xa)
            y = selective_scan(xa, delta, self.a, b_vec, c_vec, None, z, None, True, self.recompute_scan)
        return self.out_proj(y)

    def parameters(self):
        if self.tp is not None:
            return [self.in_proj, self.conv_weight, self.a, self.x_proj, self.out_proj, self.dt_up, self.dt_bias, self.d_skip, self.conv_bias]
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
    """Token embedding -> num_layers x (LayerNorm -> MambaBlock(standard) -> residual) -> LayerNorm -> LM head.

    With `tp` (a `parallel.tp.TPContext`) the blocks are tensor-parallel and everything between them is sequence
    parallel: each rank embeds, normalises and scores only its own rows (its own sequences of the global batch), the
    loss is the mean over the ranks' local means, and `make_optimizer` pairs a local Adam for the channel-sharded
    parameters with a sharded `DistributedAdam(average=False)` for the replicated ones (embedding, norms, head), whose
    per-rank gradients are partial sums over that rank's rows."""

    def __init__(self, vocab: int, d_model: int, num_layers: int, d_state: int = 16, d_conv: int = 4, expand: int = 2,
                 dt_rank: int = 0, init_std: float = 0.02, tp=None, seed: int = 1234, recompute_scan: bool = False):
        init = nn.normal_init(init_std)
        self.tp = tp
        g = torch.Generator().manual_seed(seed) if tp is not None else None
        self.tok = nn.Embedding(vocab, d_model, std=init_std)
        self.norms = [nn.LayerNorm(d_model) for _ in range(num_layers)]
        self.blocks = [MambaBlock(d_model, d_state, expand, d_conv, standard=True, dt_rank=dt_rank, init=init, tp=tp, generator=g)
                       for _ in range(num_layers)]
        for b in self.blocks:
            b.recompute_scan = recompute_scan
        self.ln_final = nn.LayerNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab, bias=False, init=init)

    def children(self):
        return [self.tok] + self.norms + self.blocks + [self.ln_final, self.lm_head]

    def hidden(self, ids):
        h = self.tok(ids)
        if self.tp is not None:
            Bl, S, d = h.shape
            h = h.reshape(Bl * S, d)                                   # this rank's rows
            for i, (n, b) in enumerate(zip(self.norms, self.blocks)):
                h = mark(h, i + 1)
                h = b.forward_tp(n(h), S, residual=h)
            return self.ln_final(mark(h, len(self.blocks) + 1)).view(Bl, S, d)
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
        l = lm_head_ce(self.hidden(ids), self.lm_head.weight, None, labels)
        if self.tp is not None and self.tp.world > 1:
            from ..parallel.tp import scale_grad
            l = scale_grad(l, 1.0 / self.tp.world)                     # the job's loss is the mean over the ranks' local means
        return l

    def make_optimizer(self, lr: float = 1e-3, **kw):
        """The optimizer that matches this model's parallel layout."""
        from ..optim import Adam, MultiOptimizer
        if self.tp is None or self.tp.world == 1:
            return Adam(self.parameters(), lr=lr, **kw)
        from ..parallel.ddp import DistributedAdam
        sharded = [p for p in self.parameters() if getattr(p, "_tp_sharded", False)]
        shared = [p for p in self.parameters() if not getattr(p, "_tp_sharded", False)]
        return MultiOptimizer([DistributedAdam(shared, lr=lr, group=self.tp.group, average=False,
                                               mode="fused" if self.tp.backend == "fused" else "nccl", **kw),
                               Adam(sharded, lr=lr, **kw)])

    def parameters(self):
        ps = self.tok.parameters()
        for n, b in zip(self.norms, self.blocks):
            ps += n.parameters() + b.parameters()
        return ps + self.ln_final.parameters() + self.lm_head.parameters()


from .._compat import alias_fields as _alias_fields  # noqa: E402

_alias_fields(Mamba, d_model=lambda self: self.blocks[0].d_model)          # src/mamba.rs:137-141
