"""Library baseline of the FineGrainedMoE transformer LM configuration: stock PyTorch only.

cuBLAS GEMMs (`F.linear`), `scaled_dot_product_attention`, `nn.LayerNorm`, `F.cross_entropy`, fused `torch.optim.Adam`,
and for expert parallelism the textbook NCCL recipe: sort the (token, choice) pairs by expert, exchange counts,
`all_to_all_single` the rows to the owning ranks, run each local expert with cuBLAS, `all_to_all_single` back, weight and
sum; the shared (non-expert) parameters are data-parallel through one flat NCCL all-reduce per step. None of this
package's kernels are on this path: it is the number the peer-memory dispatch / combine kernels and the tcgen05 expert
GEMMs are measured against. Same architecture as `rust_neural_network_b200.models.moe.MoETransformerLM` (softmax router,
top-k with renormalised weights, aux load-balance loss, `num_shared` shared experts, SiLU experts, no capacity drops).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as tnn
import torch.nn.functional as TF


class _A2A(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.cfg = (send, recv, group)
        out = x.new_empty((sum(recv),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        send, recv, group = ctx.cfg
        out = g.new_empty((sum(send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=send, input_split_sizes=recv, group=group)
        return out, None, None, None


class Expert(tnn.Module):
    def __init__(self, d, hid):
        super().__init__()
        self.l1, self.l2 = tnn.Linear(d, hid), tnn.Linear(hid, d)

    def forward(self, x):
        return self.l2(TF.silu(self.l1(x)))


class MoE(tnn.Module):
    def __init__(self, d, hid, E, k, num_shared, world, rank, group, aux_coef=0.01):
        super().__init__()
        self.E, self.k, self.world, self.rank, self.group, self.aux_coef = E, k, world, rank, group, aux_coef
        self.E_local = E // world
        self.gate = tnn.Linear(d, E)
        self.shared = tnn.ModuleList(Expert(d, hid) for _ in range(num_shared))
        self.experts = tnn.ModuleList(Expert(d, hid) for _ in range(self.E_local))
        for p in self.experts.parameters():
            p.ep_owned = True
        self.aux = None

    def forward(self, x):
        T, d = x.shape
        out = sum(s(x) for s in self.shared)
        probs = torch.softmax(self.gate(x).float(), -1)
        w, idx = torch.topk(probs, self.k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        flat_e = idx.reshape(-1)
        counts = torch.bincount(flat_e, minlength=self.E)
        f = counts.float() / float(T * self.k)
        self.aux = self.aux_coef * self.E * (f * probs.mean(0)).sum()
        order = torch.argsort(flat_e, stable=True)
        tok = torch.div(order, self.k, rounding_mode="floor")
        rows = (x.to(torch.bfloat16) if x.is_cuda else x)[tok]        # bf16 rows on the wire, like the kernels this is compared with
        if self.world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)
            send = counts.view(self.world, self.E_local).sum(1).tolist()
            rc = recv_counts.view(self.world, self.E_local)
            recv = rc.sum(1).tolist()
            rows = _A2A.apply(rows, send, recv, self.group)
            src_e = torch.repeat_interleave(torch.arange(self.world * self.E_local, device=x.device) % self.E_local, rc.reshape(-1))
            by_e = torch.argsort(src_e, stable=True)
            rows = rows[by_e]
            per_e = rc.sum(0).tolist()
        else:
            per_e = counts.tolist()
        outs, off = [], 0
        for e, n in enumerate(per_e):
            outs.append(self.experts[e](rows[off:off + n]))
            off += n
        y = torch.cat(outs, 0)
        if self.world > 1:
            y = torch.empty_like(y).index_copy(0, by_e, y)
            y = _A2A.apply(y, recv, send, self.group)
        contrib = (y.float() * w.reshape(-1)[order].float().unsqueeze(1)).to(x.dtype)
        return out + torch.zeros_like(x).index_add(0, tok, contrib)


class Layer(tnn.Module):
    def __init__(self, d, heads, hid, E, k, num_shared, world, rank, group):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = tnn.LayerNorm(d), tnn.LayerNorm(d)
        self.qkv, self.o = tnn.Linear(d, 3 * d), tnn.Linear(d, d)
        self.moe = MoE(d, hid, E, k, num_shared, world, rank, group)

    def forward(self, x):
        B, S, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = TF.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, d))
        return x + self.moe(self.ln2(x).reshape(B * S, d)).view(B, S, d)


class TorchMoELM(tnn.Module):
    def __init__(self, vocab, d, layers, heads, E, k, num_shared, hid, max_seq, world=1, rank=0, group=None, init_std=0.02):
        super().__init__()
        self.tok, self.pos = tnn.Embedding(vocab, d), tnn.Embedding(max_seq, d)
        self.layers = tnn.ModuleList(Layer(d, heads, hid, E, k, num_shared, world, rank, group) for _ in range(layers))
        self.ln_final = tnn.LayerNorm(d)
        self.lm_head = tnn.Linear(d, vocab, bias=False)
        for m in self.modules():
            if isinstance(m, (tnn.Linear, tnn.Embedding)):
                tnn.init.normal_(m.weight, std=init_std)
            if isinstance(m, tnn.Linear) and m.bias is not None:
                tnn.init.zeros_(m.bias)

    def forward(self, ids, labels):
        B, S = ids.shape
        h = self.tok(ids) + self.pos(torch.arange(S, device=ids.device))
        aux = 0.0
        for layer in self.layers:
            h = layer(h)
            aux = aux + layer.moe.aux
        logits = self.lm_head(self.ln_final(h))
        return TF.cross_entropy(logits.float().view(B * S, -1), labels.view(-1)) + aux


class TorchMoEStep:
    """One training step: autocast bf16 forward / backward, one flat all-reduce of the shared parameters' gradients,
    fused Adam. Eager (the split sizes of the all-to-alls are read on the host)."""

    def __init__(self, model, world, group=None, lr=1e-3):
        self.model, self.world, self.group = model, world, group
        self.shared = [p for p in model.parameters() if not getattr(p, "ep_owned", False)]
        self.owned = [p for p in model.parameters() if getattr(p, "ep_owned", False)]
        n = sum(p.numel() for p in self.shared)
        self.flat_grad = torch.zeros(n, device=self.shared[0].device)
        off = 0
        for p in self.shared:
            p.grad = self.flat_grad[off:off + p.numel()].view_as(p)
            off += p.numel()
        self.opt = torch.optim.Adam(model.parameters(), lr=lr, fused=True)

    def step(self, ids, labels):
        self.flat_grad.zero_()
        for p in self.owned:
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.model(ids, labels)
        loss.backward()
        if self.world > 1:
            dist.all_reduce(self.flat_grad, group=self.group)
            self.flat_grad.mul_(1.0 / self.world)
            for p in self.owned:
                if p.grad is not None:
                    p.grad.mul_(1.0 / self.world)
        self.opt.step()
        return loss.detach()
