"""Mixture-of-experts layers (rust-nn src/nn.rs:397-497) with real routing, and the MoE transformer LM.

`NormalMoE(in, hidden, E)` and `FineGrainedMoE(in, shared_hidden, expert_hidden, E)` keep the
reference constructors and parameter order (gate, [shared expert], experts; each expert
Linear -> act -> Linear with biases). The reference computes gate logits and then ignores them,
summing all experts densely; `routing="dense"` reproduces that. The default `routing="topk"` is a
softmax router with top-k selection, capacity-bounded dispatch, batched expert GEMMs and a weighted
combine, plus the auxiliary load-balance loss  E * sum_e f_e * P_e  (f_e: fraction of routed
assignments that went to expert e, P_e: mean router probability of e), exposed as `last_aux_loss`.

Kernels: router forward/backward, dispatch (atomic slot claim + row copy), combine and their
adjoints (csrc/moe/moe.cu); the experts run as two batched calls of the tcgen05 GEMM with a
per-expert bias and the activation fused in the epilogue. With expert parallelism (`ep_group`) every
rank owns E/world experts; dispatch writes token rows straight into the owning rank's capacity
buffer and combine reads the expert outputs back from it over NVLink peer memory, so the two
all-to-alls are the kernels' own remote stores / loads.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional

import torch
from torch.autograd import Function

from .. import _native as nv
from .. import nn
from ..ops import functional as F
from ..ops.gemm import gemm

_P = C.c_void_p
nv.register_sigs({
    "b200_router_fwd": [_P, _P, _P, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, _P],
    "b200_router_bwd": [_P, _P, _P, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, _P],
    "b200_moe_dispatch": [_P, _P, _P, C.POINTER(_P), C.POINTER(_P), C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, _P],
    "b200_moe_combine_fwd": [C.POINTER(_P), C.c_int, _P, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_longlong, _P],
    "b200_moe_combine_bwd": [C.POINTER(_P), C.POINTER(_P), C.c_int, _P, _P, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_longlong, _P],
    "b200_moe_gather_sum": [C.POINTER(_P), C.c_int, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_longlong, _P],
})


def _ptr_array(ptrs):
    return (_P * len(ptrs))(*ptrs)


# ----------------------------------------------------------------------------- router
def router_ref(logits, k, renorm):
    p = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(p, k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx.int(), w, p


class RouterFn(Function):
    """logits [T, E] -> (idx [T, k] int32, weights [T, k] fp32, counts [E] int32, aux_loss 0-d)."""

    @staticmethod
    def forward(ctx, logits, k, renorm, aux_coef):
        T, E = logits.shape
        if logits.is_cuda:
            lg = logits.contiguous()
            idx = torch.empty((T, k), dtype=torch.int32, device=lg.device)
            w = torch.empty((T, k), dtype=torch.float32, device=lg.device)
            probs = torch.empty((T, E), dtype=torch.float32, device=lg.device)
            counts = torch.zeros(E, dtype=torch.int32, device=lg.device)
            nv.check(nv.cuda().b200_router_fwd(lg.data_ptr(), idx.data_ptr(), w.data_ptr(), probs.data_ptr(), counts.data_ptr(), T, E, k,
                                               int(renorm), 1 if lg.dtype == torch.bfloat16 else 0, nv.stream_ptr()), "router_fwd")
            nv.count_launch()
        else:
            idx, w, probs = router_ref(logits, k, renorm)
            counts = torch.bincount(idx.reshape(-1).long(), minlength=E).int()
        f = counts.float() / float(T * k)
        aux = E * (f * probs.mean(0)).sum()
        ctx.save_for_backward(idx, probs, f)
        ctx.cfg = (k, renorm, aux_coef, logits.dtype)
        ctx.mark_non_differentiable(idx, counts)
        return idx, w, counts, aux

    @staticmethod
    def backward(ctx, _gi, dw, _gc, daux):
        idx, probs, f = ctx.saved_tensors
        k, renorm, aux_coef, dtype = ctx.cfg
        T, E = probs.shape
        aux_g = None
        if daux is not None:
            aux_g = (daux.float() * E / T) * f                    # d aux / d probs[t, e] (f_e is treated as a constant)
        if dw is None:
            dw = torch.zeros((T, k), dtype=torch.float32, device=probs.device)
        if probs.is_cuda:
            dlog = torch.empty((T, E), dtype=dtype, device=probs.device)
            dwc = dw.float().contiguous()
            ag = aux_g.contiguous() if aux_g is not None else None
            nv.check(nv.cuda().b200_router_bwd(dwc.data_ptr(), idx.data_ptr(), probs.data_ptr(), nv.ptr(ag), dlog.data_ptr(), T, E, k,
                                               int(renorm), 1 if dtype == torch.bfloat16 else 0, nv.stream_ptr()), "router_bwd")
            nv.count_launch()
            return dlog, None, None, None
        g = torch.zeros_like(probs) if aux_g is None else aux_g.expand(T, E).clone()
        sel = probs.gather(1, idx.long())
        if renorm:
            s = sel.sum(-1, keepdim=True)
            dot = (dw * sel / s).sum(-1, keepdim=True)
            d = (dw - dot) / s
        else:
            d = dw
        g.scatter_add_(1, idx.long(), d.float())
        dlog = probs * (g - (probs * g).sum(-1, keepdim=True))
        return dlog.to(dtype), None, None, None


# ----------------------------------------------------------------------------- dispatch / experts / combine
class EPContext:
    """Symmetric (peer-mapped) buffers of an expert-parallel group. `world == 1` needs no peers."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self._bufs = {}

    def buffer(self, key, numel, dtype, device):
        """A zero-initialisable buffer mapped by every rank: returns (local tensor, [address on each rank])."""
        k = (key, numel, dtype)
        if k not in self._bufs:
            if self.world == 1:
                t = torch.empty(numel, dtype=dtype, device=device)
                self._bufs[k] = (t, [t.data_ptr()])
            else:
                from ..parallel.ddp import SymmetricBuffer
                sb = SymmetricBuffer(numel, dtype, device, self.group)
                self._bufs[k] = (sb.tensor, sb.ptrs, sb)
        e = self._bufs[k]
        return e[0], e[1]

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(self.group)


class MoEExpertsFn(Function):
    """Routed experts: out[t] = sum_j w[t,j] * FFN_{idx[t,j]}(x[t]).  x [T, d] bf16 (CUDA)."""

    @staticmethod
    def forward(ctx, x, idx, w, W1, b1, W2, b2, act, cap, ep: Optional[EPContext]):
        T, d = x.shape
        k = idx.shape[1]
        E_local, hid = W1.shape[0], W1.shape[1]
        world = ep.world if ep is not None else 1
        rows = E_local * cap
        dev = x.device
        ep = ep or _LOCAL_EP
        xbuf, xptrs = ep.buffer("x", rows * d, torch.bfloat16, dev)
        fill, fptrs = ep.buffer("fill", max(E_local, 4), torch.int32, dev)
        ybuf, yptrs = ep.buffer("y", rows * d, torch.bfloat16, dev)
        xbuf.zero_(); fill.zero_()
        ep.barrier()                                              # every rank's buffers are cleared before anyone writes
        dest = torch.empty((T, k), dtype=torch.int32, device=dev)
        lib = nv.cuda()
        xc = x.contiguous()
        nv.check(lib.b200_moe_dispatch(xc.data_ptr(), idx.data_ptr(), dest.data_ptr(), _ptr_array(xptrs), _ptr_array(fptrs), world,
                                       T, k, d, E_local, cap, nv.stream_ptr()), "moe_dispatch")
        ep.barrier()                                              # all remote rows have landed
        xb = xbuf.view(E_local, cap, d)
        W1l, W2l = F.lp(W1), F.lp(W2)
        h, pre = gemm(xb, W1l, bias=b1.detach() if b1 is not None else None, act=act, want_aux=True)        # [E, cap, hid]
        y = gemm(h, W2l, bias=b2.detach() if b2 is not None else None)                                       # [E, cap, d]
        ybuf.view(E_local, cap, d).copy_(y)
        ep.barrier()
        out = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
        wc = w.float().contiguous()
        nv.check(lib.b200_moe_combine_fwd(_ptr_array(yptrs), world, dest.data_ptr(), wc.data_ptr(), out.data_ptr(), T, k, d, rows,
                                          nv.stream_ptr()), "moe_combine_fwd")
        nv.count_launch(2)
        ep.barrier()
        ctx.save_for_backward(dest, wc, xb.clone(), h, pre, y, W1, b1, W2, b2)
        ctx.cfg = (act, cap, ep, T, d, k, E_local, hid)
        return out

    @staticmethod
    def backward(ctx, dout):
        dest, wc, xb, h, pre, y, W1, b1, W2, b2 = ctx.saved_tensors
        act, cap, ep, T, d, k, E_local, hid = ctx.cfg
        world, rows, dev = ep.world, E_local * cap, dout.device
        lib = nv.cuda()
        ybuf, yptrs = ep.buffer("y", rows * d, torch.bfloat16, dev)
        dybuf, dyptrs = ep.buffer("dy", rows * d, torch.bfloat16, dev)
        ybuf.view(E_local, cap, d).copy_(y)
        dybuf.zero_()
        ep.barrier()
        dw = torch.empty((T, k), dtype=torch.float32, device=dev)
        dc = dout.contiguous()
        nv.check(lib.b200_moe_combine_bwd(_ptr_array(yptrs), _ptr_array(dyptrs), world, dest.data_ptr(), wc.data_ptr(), dc.data_ptr(),
                                          dw.data_ptr(), T, k, d, rows, nv.stream_ptr()), "moe_combine_bwd")
        ep.barrier()
        dy = dybuf.view(E_local, cap, d)
        W1l, W2l = F.lp(W1), F.lp(W2)
        dh = gemm(dy, W2l, b_mn=True, aux_in=pre, dact=act)                                   # [E, cap, hid]
        dW2 = gemm(dy, h, a_mn=True, b_mn=True, out_dtype=torch.float32)                       # [E, d, hid]
        dW1 = gemm(dh, xb, a_mn=True, b_mn=True, out_dtype=torch.float32)                      # [E, hid, d]
        dxb = gemm(dh, W1l, b_mn=True)                                                         # [E, cap, d]
        db1 = db2 = None
        if b1 is not None:
            db1 = torch.zeros((E_local, hid), dtype=torch.float32, device=dev)
            nv.check(lib.b200_colsum_batched(dh.data_ptr(), db1.data_ptr(), E_local, cap, hid, hid, cap * hid, 1, nv.stream_ptr()), "colsum_batched")
        if b2 is not None:
            db2 = torch.zeros((E_local, d), dtype=torch.float32, device=dev)
            nv.check(lib.b200_colsum_batched(dy.data_ptr(), db2.data_ptr(), E_local, cap, d, d, cap * d, 1, nv.stream_ptr()), "colsum_batched")
        # adjoint of dispatch: pull the token gradients back from the owning ranks (reuses the "x" buffer)
        xbuf, xptrs = ep.buffer("x", rows * d, torch.bfloat16, dev)
        xbuf.view(E_local, cap, d).copy_(dxb)
        ep.barrier()
        dx = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
        nv.check(lib.b200_moe_gather_sum(_ptr_array(xptrs), world, dest.data_ptr(), dx.data_ptr(), T, k, d, rows, nv.stream_ptr()), "moe_gather_sum")
        nv.count_launch(4)
        ep.barrier()
        return dx, None, dw, dW1, db1, dW2, db2, None, None, None


_LOCAL_EP = EPContext(None) if True else None


def moe_experts_ref(x, idx, w, W1, b1, W2, b2, act):
    """Dense per-token loop over the selected experts (fp32): the oracle of the routed path (no capacity drops)."""
    from ..ops.gemm import act_ref
    xf = x.float()
    out = torch.zeros_like(xf)
    for j in range(idx.shape[1]):
        e = idx[:, j].long()
        h = torch.einsum("td,thd->th", xf, W1.float()[e]) + (b1.float()[e] if b1 is not None else 0)
        h = act_ref(h, act)
        y = torch.einsum("th,tdh->td", h, W2.float()[e]) + (b2.float()[e] if b2 is not None else 0)
        out = out + w[:, j:j + 1].float() * y
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- modules
class _Expert(nn.Module):
    def __init__(self, d_in, hidden, act, init):
        self.l1 = nn.Linear(d_in, hidden, init=init)
        self.l2 = nn.Linear(hidden, d_in, init=init)
        self.act = act

    def forward(self, x):
        return self.l2(F.linear(x, self.l1.weight, self.l1.bias, self.act, None))

    def parameters(self):
        return self.l1.parameters() + self.l2.parameters()


class _RoutedMoE(nn.Module):
    """Shared machinery of NormalMoE / FineGrainedMoE."""

    def __init__(self, d_in, expert_hidden, num_experts, top_k, act, routing, capacity_factor, aux_coef, renorm, init,
                 shared_hidden=0, num_shared=0, ep_group=None):
        self.d_in, self.E, self.top_k, self.act, self.routing = d_in, num_experts, min(top_k, num_experts), act, routing
        self.capacity_factor, self.aux_coef, self.renorm = capacity_factor, aux_coef, renorm
        self.gate = nn.Linear(d_in, num_experts, init=init)
        self.shared = [_Expert(d_in, shared_hidden, act, init) for _ in range(num_shared)]
        self.ep = EPContext(ep_group) if ep_group is not None else None
        world = self.ep.world if self.ep is not None else 1
        assert num_experts % world == 0
        self.E_local = num_experts // world
        # experts are stored stacked ([E_local, hidden, d] ...) so they run as batched GEMMs; the per-expert
        # tensors of the reference layout are views produced by `checkpoint_tensors()`
        std_like = lambda *s: init(s)
        self.W1 = nn._param(torch.stack([init((expert_hidden, d_in)) for _ in range(self.E_local)]))
        self.b1 = nn._param(torch.zeros(self.E_local, expert_hidden))
        self.W2 = nn._param(torch.stack([init((d_in, expert_hidden)) for _ in range(self.E_local)]))
        self.b2 = nn._param(torch.zeros(self.E_local, d_in))
        self.last_aux_loss = None
        self.last_counts = None

    def children(self):
        return [self.gate] + list(self.shared)

    def parameters(self):
        ps = self.gate.parameters()
        for s in self.shared:
            ps += s.parameters()
        return ps + [self.W1, self.b1, self.W2, self.b2]

    def checkpoint_tensors(self):
        """Tensors in the reference's order: gate, shared experts, then per expert (W1, b1, W2, b2)."""
        ts = self.gate.parameters()
        for s in self.shared:
            ts += s.parameters()
        for e in range(self.E_local):
            ts += [self.W1[e], self.b1[e], self.W2[e], self.b2[e]]
        return ts

    def capacity(self, tokens: int) -> int:
        world = self.ep.world if self.ep is not None else 1
        c = math.ceil(self.capacity_factor * tokens * world * self.top_k / self.E)
        return max(128, (c + 127) // 128 * 128)

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, self.d_in)
        out = None
        for s in self.shared:
            o = s(x2)
            out = o if out is None else F_add(out, o)
        if self.routing == "dense":
            # reference behaviour: gate logits are computed and ignored, all experts are summed
            _ = self.gate(x2)
            for e in range(self.E_local):
                h = F.linear(x2, self.W1[e], self.b1[e], self.act, None)
                o = F.linear(h, self.W2[e], self.b2[e], "none", None)
                out = o if out is None else F_add(out, o)
            self.last_aux_loss = None
            return out.reshape(shape)
        logits = self.gate(x2)
        idx, w, counts, aux = RouterFn.apply(logits, self.top_k, self.renorm, self.aux_coef)
        self.last_aux_loss = aux * self.aux_coef
        self.last_counts = counts
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            routed = MoEExpertsFn.apply(x2, idx, w, self.W1, self.b1, self.W2, self.b2, self.act, self.capacity(x2.shape[0]), self.ep)
        else:
            routed = _experts_dense_autograd(x2, idx, w, self.W1, self.b1, self.W2, self.b2, self.act)
        out = routed if out is None else F_add(out, routed)
        return out.reshape(shape)


def _experts_dense_autograd(x, idx, w, W1, b1, W2, b2, act):
    """Differentiable fp32/CPU path: the per-token expert loop written with plain tensor ops."""
    from ..ops.gemm import act_ref
    xf = x.float()
    out = 0
    for j in range(idx.shape[1]):
        e = idx[:, j].long()
        h = act_ref(torch.einsum("td,thd->th", xf, W1.float()[e]) + b1.float()[e], act)
        y = torch.einsum("th,tdh->td", h, W2.float()[e]) + b2.float()[e]
        out = out + w[:, j:j + 1].float() * y
    return out.to(x.dtype)


def F_add(a, b):
    from .looped_transformer import _add
    return _add(a, b)


class NormalMoE(_RoutedMoE):
    """`NormalMoE::new(in, hidden, E)` (src/nn.rs:397-434): gate Linear(in, E), experts Linear -> ReLU -> Linear."""

    def __init__(self, in_features: int, hidden_features: int, num_experts: int, top_k: int = 2, routing: str = "topk",
                 act: str = "relu", capacity_factor: float = 1.5, aux_coef: float = 0.01, renorm: bool = True,
                 init=nn.he_normal, ep_group=None):
        super().__init__(in_features, hidden_features, num_experts, top_k, act, routing, capacity_factor, aux_coef, renorm, init,
                         ep_group=ep_group)


class FineGrainedMoE(_RoutedMoE):
    """`FineGrainedMoE::new(in, shared_hidden, expert_hidden, E)` (src/nn.rs:445-496): gate, one shared expert
    (`num_shared` generalises it), E small routed experts."""

    def __init__(self, in_features: int, shared_hidden: int, expert_hidden: int, num_experts: int, top_k: int = 6,
                 num_shared: int = 1, routing: str = "topk", act: str = "relu", capacity_factor: float = 1.25,
                 aux_coef: float = 0.01, renorm: bool = True, init=nn.he_normal, ep_group=None):
        super().__init__(in_features, expert_hidden, num_experts, top_k, act, routing, capacity_factor, aux_coef, renorm, init,
                         shared_hidden=shared_hidden, num_shared=num_shared, ep_group=ep_group)


class MoETransformerLM(nn.Module):
    """Token embedding -> L x (LN -> causal MHA -> residual; LN -> FineGrainedMoE -> residual) -> LN -> LM head.
    The loss adds the routers' load-balance terms."""

    def __init__(self, vocab: int, d_model: int, layers: int, heads: int, num_experts: int, top_k: int, num_shared: int,
                 expert_hidden: int, max_seq: int, init_std: float = 0.02, ep_group=None, act: str = "silu"):
        from .looped_transformer import MultiHeadAttention
        init = nn.normal_init(init_std)
        self.tok = nn.Embedding(vocab, d_model, std=init_std)
        self.pos = nn.Embedding(max_seq, d_model, std=init_std)
        self.ln1 = [nn.LayerNorm(d_model) for _ in range(layers)]
        self.attn = [MultiHeadAttention(d_model, heads, causal=True, init=init) for _ in range(layers)]
        self.ln2 = [nn.LayerNorm(d_model) for _ in range(layers)]
        self.moe = [FineGrainedMoE(d_model, expert_hidden, expert_hidden, num_experts, top_k=top_k, num_shared=num_shared, act=act,
                                   init=init, ep_group=ep_group) for _ in range(layers)]
        self.ln_final = nn.LayerNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab, bias=False, init=init)

    def children(self):
        return [self.tok, self.pos] + self.ln1 + self.attn + self.ln2 + self.moe + [self.ln_final, self.lm_head]

    def parameters(self):
        ps = self.tok.parameters() + self.pos.parameters()
        for a, b, c, d in zip(self.ln1, self.attn, self.ln2, self.moe):
            ps += a.parameters() + b.parameters() + c.parameters() + d.parameters()
        return ps + self.ln_final.parameters() + self.lm_head.parameters()

    def hidden(self, ids):
        from .lm import _add_rows
        B, S = ids.shape
        h = self.tok(ids)
        h = _add_rows(h, F.embedding(torch.arange(S, device=ids.device), self.pos.weight, self.compute_dtype))
        aux = None
        from ..parallel.ddp import mark
        for i, (ln1, at, ln2, moe) in enumerate(zip(self.ln1, self.attn, self.ln2, self.moe)):
            h = mark(h, i + 1)
            h = at(ln1(h), residual=h)
            h = F_add(h, moe(ln2(h)))
            if moe.last_aux_loss is not None:
                aux = moe.last_aux_loss if aux is None else aux + moe.last_aux_loss
        return self.ln_final(mark(h, len(self.moe) + 1)), aux

    def dp_groups(self):
        """Parameter groups in forward order; `mark(h, k)` sits in front of group k."""
        layers = [a.parameters() + b.parameters() + c.parameters() + d.parameters()
                  for a, b, c, d in zip(self.ln1, self.attn, self.ln2, self.moe)]
        return [self.tok.parameters() + self.pos.parameters()] + layers + [self.ln_final.parameters() + self.lm_head.parameters()]

    def loss(self, ids, labels):
        from ..ops.transformer import lm_head_ce
        h, aux = self.hidden(ids)
        l = lm_head_ce(h, self.lm_head.weight, None, labels)
        return l if aux is None else l + aux.to(l.dtype)

    def forward(self, ids):
        return self.lm_head(self.hidden(ids)[0])
