"""Library baseline of the tensor-parallel Mamba LM configuration: NCCL collectives around cuBLAS GEMMs.

Same model and the same parallel layout as `rust_neural_network_b200.models.mamba.MambaLM(tp=...)` (channel-sharded
blocks on row-sharded activations), but every projection is `F.linear` (cuBLAS), every collective is a NCCL call
(`all_gather_into_tensor` before `in_proj`, `reduce_scatter_tensor` after `out_proj`, `all_reduce` for the narrow
x-projection, one flat `all_reduce` for the replicated parameters' gradients), LayerNorm / embedding / cross-entropy /
Adam are stock PyTorch. Stock PyTorch has no selective scan or depthwise causal conv with a backward, so those two ops
are this package's kernels (`ops.scan`) in both arms; what this baseline isolates is the fused all-gather->GEMM,
GEMM->reduce-scatter and all-reduce kernels and the tcgen05 GEMMs.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as tnn
import torch.nn.functional as TF


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world):
        ctx.cfg = (group, world)
        if world == 1:
            return x
        out = x.new_empty((x.shape[0] * world,) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group, world = ctx.cfg
        if world == 1:
            return g, None, None
        out = g.new_empty((g.shape[0] // world,) + tuple(g.shape[1:]))
        dist.reduce_scatter_tensor(out, g.contiguous(), group=group)
        return out, None, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world):
        ctx.cfg = (group, world)
        if world == 1:
            return x
        out = x.new_empty((x.shape[0] // world,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group, world = ctx.cfg
        if world == 1:
            return g, None, None
        out = g.new_empty((g.shape[0] * world,) + tuple(g.shape[1:]))
        dist.all_gather_into_tensor(out, g.contiguous(), group=group)
        return out, None, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world):
        ctx.cfg = (group, world)
        if world > 1:
            x = x.clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        group, world = ctx.cfg
        if world > 1:
            g = g.clone()
            dist.all_reduce(g, group=group)
        return g, None, None


class Block(tnn.Module):
    def __init__(self, d, N, expand, Kc, R, world, rank, group, init_std, gen):
        super().__init__()
        di = expand * d
        dl = di // world
        lo, hi = rank * dl, (rank + 1) * dl
        self.dims = (d, N, R, dl)
        self.world, self.group = world, group
        rn = lambda *s: torch.randn(*s, generator=gen) * init_std
        wx, wz = rn(di, d), rn(di, d)
        self.in_proj = tnn.Parameter(torch.cat([wx[lo:hi], wz[lo:hi]], 0))
        self.conv_weight = tnn.Parameter(((torch.rand(di, Kc, generator=gen) * 2 - 1) / math.sqrt(Kc))[lo:hi].contiguous())
        self.conv_bias = tnn.Parameter(torch.zeros(dl))
        self.a_log = tnn.Parameter(torch.log(torch.arange(1, N + 1, dtype=torch.float32)).repeat(dl, 1))
        self.x_proj = tnn.Parameter(torch.cat([rn(R, di), rn(N, di), rn(N, di)], 0)[:, lo:hi].contiguous())
        self.dt_up = tnn.Parameter(((torch.rand(di, R, generator=gen) * 2 - 1) * R ** -0.5)[lo:hi].contiguous())
        dt = torch.exp(torch.rand(di, generator=gen) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp_min(1e-4)
        self.dt_bias = tnn.Parameter((dt + torch.log(-torch.expm1(-dt)))[lo:hi].contiguous())
        self.d_skip = tnn.Parameter(torch.ones(dl))
        self.out_proj = tnn.Parameter(rn(d, di)[:, lo:hi].contiguous())
        for p in self.parameters():
            p.tp_owned = True

    def forward(self, x_s, S):
        from rust_neural_network_b200.ops.scan import causal_conv1d, selective_scan
        d, N, R, dl = self.dims
        bf = torch.bfloat16
        xz = TF.linear(_AllGatherRows.apply(x_s, self.group, self.world), self.in_proj.to(bf))
        M = xz.shape[0]
        Bt = M // S
        xs, z = xz[:, :dl].view(Bt, S, dl), xz[:, dl:].view(Bt, S, dl)
        xa = causal_conv1d(xs, self.conv_weight, self.conv_bias, "silu")
        xp = _AllReduce.apply(TF.linear(xa.view(M, dl), self.x_proj.to(bf)).float(), self.group, self.world).to(bf)
        dt = TF.linear(xp[:, :R], self.dt_up.to(bf))
        y = selective_scan(xa, dt.view(Bt, S, dl), -torch.exp(self.a_log.float()), xp[:, R:R + N].view(Bt, S, N),
                           xp[:, R + N:].view(Bt, S, N), self.d_skip, z, self.dt_bias, True)
        return _ReduceScatterRows.apply(TF.linear(y.reshape(M, dl), self.out_proj.to(bf)), self.group, self.world)


class TorchMambaLM(tnn.Module):
    def __init__(self, vocab, d, layers, d_state, d_conv, expand, dt_rank, world=1, rank=0, group=None, init_std=0.02, seed=1234):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.world = world
        self.tok = tnn.Embedding(vocab, d)
        tnn.init.normal_(self.tok.weight, std=init_std)
        self.norms = tnn.ModuleList(tnn.LayerNorm(d) for _ in range(layers))
        self.blocks = tnn.ModuleList(Block(d, d_state, expand, d_conv, dt_rank, world, rank, group, init_std, gen) for _ in range(layers))
        self.ln_final = tnn.LayerNorm(d)
        self.lm_head = tnn.Linear(d, vocab, bias=False)
        tnn.init.normal_(self.lm_head.weight, std=init_std)

    def forward(self, ids, labels):
        Bl, S = ids.shape
        h = self.tok(ids).to(torch.bfloat16).view(Bl * S, -1)
        for n, b in zip(self.norms, self.blocks):
            h = h + b(TF.layer_norm(h.float(), n.normalized_shape, n.weight, n.bias, n.eps).to(torch.bfloat16), S)
        hf = TF.layer_norm(h.float(), self.ln_final.normalized_shape, self.ln_final.weight, self.ln_final.bias, self.ln_final.eps)
        logits = TF.linear(hf.to(torch.bfloat16), self.lm_head.weight.to(torch.bfloat16))
        return TF.cross_entropy(logits.float(), labels.view(-1))


class TorchMambaStep:
    """One training step: forward / backward of this rank's rows, one flat NCCL all-reduce (sum) of the replicated
    parameters' gradients, fused Adam on everything. Each rank's loss is scaled by 1/world, so the job's loss is the
    mean over the ranks' local means and the channel-sharded parameters need no reduction."""

    def __init__(self, model, world, group=None, lr=1e-3):
        self.model, self.world, self.group = model, world, group
        self.shared = [p for p in model.parameters() if not getattr(p, "tp_owned", False)]
        n = sum(p.numel() for p in self.shared)
        self.flat_grad = torch.zeros(n, device=self.shared[0].device)
        off = 0
        for p in self.shared:
            p.grad = self.flat_grad[off:off + p.numel()].view_as(p)
            off += p.numel()
        self.owned = [p for p in model.parameters() if getattr(p, "tp_owned", False)]
        self.opt = torch.optim.Adam(model.parameters(), lr=lr, fused=True)

    def step(self, ids, labels):
        self.flat_grad.zero_()
        for p in self.owned:
            p.grad = None
        loss = self.model(ids, labels)
        (loss / self.world).backward()
        if self.world > 1:
            dist.all_reduce(self.flat_grad, group=self.group)
        self.opt.step()
        return loss.detach()
