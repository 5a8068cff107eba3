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
import os
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
    "b200_ep_barrier": [C.POINTER(_P), C.c_int, C.c_int, _P, C.c_longlong, _P, _P],
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
    """Symmetric (peer-mapped) buffers of an expert-parallel group. `world == 1` needs no peers.

    The phases of a layer (dispatch -> expert GEMMs -> combine, and their adjoints) are separated by `barrier()`: with
    `backend="fused"` a one-block kernel that exchanges epoch flags with every peer on the stream (bounded wait, status
    word), so an expert-parallel step has no host synchronisation and can be captured into a CUDA graph;
    `backend="nccl"` uses a host barrier (the baseline the device protocol replaced)."""

    def __init__(self, group=None, backend: str = "fused", wait_seconds: float = 2.0):
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.backend = backend
        self.wait_seconds = wait_seconds
        self._bufs = {}
        self._bar = None
        self.clean = {}          # buffer key -> True while the buffer is known to be all zero on every rank

    def buffer(self, key, numel, dtype, device):
        """A zero-initialisable buffer mapped by every rank: returns (local tensor, [address on each rank])."""
        k = (key, numel, dtype)
        if k not in self._bufs:
            if self.world == 1:
                t = torch.zeros(numel, dtype=dtype, device=device)
                self._bufs[k] = (t, [t.data_ptr()])
            else:
                from ..parallel.ddp import SymmetricBuffer
                sb = SymmetricBuffer(numel, dtype, device, self.group)
                self._bufs[k] = (sb.tensor, sb.ptrs, sb)
            self.clean[k] = True
        e = self._bufs[k]
        return e[0], e[1]

    def _barrier_state(self, device):
        """(flag addresses on every rank, local epoch words, wait budget in cycles) of the device-side barrier; one set per
        context, shared by the barrier kernel and by the barriers inside the fused layer kernel."""
        if self._bar is None:
            hz = torch.cuda.get_device_properties(device).clock_rate * 1000
            words = torch.zeros(4, dtype=torch.int32, device=device)
            if self.world == 1:
                flags = torch.zeros(64, dtype=torch.int32, device=device)
                self._bar = (flags, [flags.data_ptr()], words, int(self.wait_seconds * hz))
            else:
                from ..parallel.ddp import SymmetricBuffer
                flags = SymmetricBuffer(64, torch.int32, device, self.group, name="ep_barrier_flags")
                import torch.distributed as dist
                dist.barrier(self.group)
                torch.cuda.synchronize()
                self._bar = (flags, flags.ptrs, words, int(self.wait_seconds * hz))
        return self._bar[1], self._bar[2], self._bar[3]

    def fused_sync(self, device):
        """Local words of the fused layer kernel's grid barrier: [0] CTA arrivals, [1] generation."""
        if getattr(self, "_sync", None) is None:
            self._sync = torch.zeros(4, dtype=torch.int32, device=device)
        return self._sync

    def barrier(self, device=None):
        if self.world == 1:
            return
        if self.backend != "fused":
            import torch.distributed as dist
            torch.cuda.current_stream().synchronize()
            dist.barrier(self.group)
            return
        ptrs, words, cycles = self._barrier_state(device)
        nv.check(nv.cuda().b200_ep_barrier(_ptr_array(ptrs), self.world, self.rank, words.data_ptr(), cycles,
                                           nv.status_word(device).data_ptr(), nv.stream_ptr()), "ep_barrier")
        nv.count_launch()


_FUSED_LAYER = os.environ.get("B200NN_MOE_FUSED_LAYER", "1") != "0"


class MoeFusedArgs(C.Structure):
    """Mirror of `MoeFusedArgs` in csrc/gemm/gemm_sm100.cu (the one-kernel forward of an expert-parallel layer)."""
    _fields_ = [("x", C.c_void_p), ("idx", C.c_void_p), ("dest", C.c_void_p),
                ("xbuf", C.c_void_p * 8), ("fill", C.c_void_p * 8), ("ybuf", C.c_void_p * 8), ("bar_flags", C.c_void_p * 8),
                ("bar_words", C.c_void_p), ("sync", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p), ("xsave", C.c_void_p),
                ("counts_out", C.c_void_p), ("tokens", C.c_longlong), ("rows_per_rank", C.c_longlong), ("wait_cycles", C.c_longlong),
                ("k", C.c_int), ("d", C.c_int), ("E_local", C.c_int), ("cap", C.c_int), ("rank", C.c_int), ("world", C.c_int),
                ("status", C.c_void_p)]


def _fused_layer_forward(ep, xc, idx, w, W1, b1, W2, b2, act, cap, xbuf, xptrs, fill, fptrs, ybuf, yptrs, dest):
    """Forward of the routed experts as ONE kernel launch: dispatch, cross-rank barrier, both grouped GEMMs over the real
    per-expert counts, barrier, combine, clearing of the input buffer, closing barrier (csrc/gemm/gemm_sm100.cu:
    moe_fused_fwd_kernel). Returns the output and the tensors the backward needs."""
    from ..ops.gemm import _num_sms
    T, d = xc.shape
    k = idx.shape[1]
    E_local, hid = W1.shape[0], W1.shape[1]
    dev = xc.device
    xb = xbuf.view(E_local, cap, d)
    fill_l = fill[:E_local]
    g1, bn1, h, pre, keep1 = gemm(xb, F.lp(W1), bias=b1.detach() if b1 is not None else None, act=act, want_aux=True, m_valid=fill_l,
                                  bn=256, _prepare=True)
    g2, bn2, _, _, keep2 = gemm(h, F.lp(W2), bias=b2.detach() if b2 is not None else None, out=ybuf.view(E_local, cap, d), m_valid=fill_l,
                                bn=256, _prepare=True)
    out = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
    xsave = torch.empty((E_local, cap, d), dtype=torch.bfloat16, device=dev)
    counts = torch.empty(E_local, dtype=torch.int32, device=dev)
    wc = w.float().contiguous()
    flag_ptrs, words, cycles = ep._barrier_state(dev)
    a = MoeFusedArgs()
    a.x, a.idx, a.dest = xc.data_ptr(), idx.data_ptr(), dest.data_ptr()
    for r in range(ep.world):
        a.xbuf[r], a.fill[r], a.ybuf[r], a.bar_flags[r] = xptrs[r], fptrs[r], yptrs[r], flag_ptrs[r]
    a.bar_words, a.sync = words.data_ptr(), ep.fused_sync(dev).data_ptr()
    a.w, a.out, a.xsave, a.counts_out = wc.data_ptr(), out.data_ptr(), xsave.data_ptr(), counts.data_ptr()
    a.tokens, a.rows_per_rank, a.wait_cycles = T, E_local * cap, cycles
    a.k, a.d, a.E_local, a.cap, a.rank, a.world = k, d, E_local, cap, ep.rank, ep.world
    a.status = nv.status_word(dev).data_ptr()
    fn = nv.cuda().b200_moe_fused_fwd
    fn.argtypes, fn.restype = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p], C.c_int
    nv.check(fn(C.addressof(g1), C.addressof(g2), C.addressof(a), _num_sms(dev), nv.stream_ptr()), "moe_fused_fwd")
    nv.count_launch()
    del keep1, keep2
    return out, (dest, wc, xsave, h, pre, W1, b1, W2, b2, counts)


class MoEExpertsFn(Function):
    """Routed experts: out[t] = sum_j w[t,j] * FFN_{idx[t,j]}(x[t]).  x [T, d] bf16 (CUDA).

    Buffer discipline (all buffers are shared by every layer of the model and live in peer-mapped memory):
      forward   entry: xbuf and fill are zero on every rank.
                dispatch (remote row stores + remote slot counters) | barrier | expert GEMMs -> ybuf | barrier |
                combine (remote row loads), then clear xbuf / fill | barrier.
      backward  entry: dybuf is zero. ybuf <- y | barrier | combine adjoint (remote loads of ybuf, remote stores into
                dybuf) | barrier | expert GEMMs, dxbuf <- d(expert input) | barrier | dispatch adjoint (remote loads of
                dxbuf), then clear dybuf.
    The closing barrier of the forward is what lets the next layer's dispatch write into a peer at once. The backward needs
    none: a peer may still be reading this rank's dxbuf when the function returns, but the next writer of dxbuf (the next
    layer's backward) first passes a barrier that every peer only reaches after it has finished that read, and dybuf is
    cleared before this rank signals that barrier."""

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
        dest = torch.empty((T, k), dtype=torch.int32, device=dev)
        lib = nv.cuda()
        xc = x.contiguous()
        if ep.backend == "fused" and x.is_cuda and _FUSED_LAYER and d % 8 == 0:
            out, saved = _fused_layer_forward(ep, xc, idx, w, W1, b1, W2, b2, act, cap, xbuf, xptrs, fill, fptrs, ybuf, yptrs, dest)
            ctx.save_for_backward(*saved)
            ctx.cfg = (act, cap, ep, T, d, k, E_local, hid)
            return out
        nv.check(lib.b200_moe_dispatch(xc.data_ptr(), idx.data_ptr(), dest.data_ptr(), _ptr_array(xptrs), _ptr_array(fptrs), world,
                                       T, k, d, E_local, cap, nv.stream_ptr()), "moe_dispatch")
        ep.barrier(dev)                                           # all remote rows have landed
        xb = xbuf.view(E_local, cap, d)
        W1l, W2l = F.lp(W1), F.lp(W2)
        # rows in use per local expert: the expert GEMMs skip the 128-row tiles past them (the capacity padding costs
        # nothing), and nothing downstream reads the rows they leave unwritten
        counts = fill[:E_local].clamp(max=cap) if x.is_cuda else None
        h, pre = gemm(xb, W1l, bias=b1.detach() if b1 is not None else None, act=act, want_aux=True, m_valid=counts)   # [E, cap, hid]
        y = gemm(h, W2l, bias=b2.detach() if b2 is not None else None, out=ybuf.view(E_local, cap, d), m_valid=counts)  # [E, cap, d], in the peers' reach
        xsave = xb.clone()
        ep.barrier(dev)                                           # every rank's expert outputs are in place
        out = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
        wc = w.float().contiguous()
        nv.check(lib.b200_moe_combine_fwd(_ptr_array(yptrs), world, dest.data_ptr(), wc.data_ptr(), out.data_ptr(), T, k, d, rows,
                                          nv.stream_ptr()), "moe_combine_fwd")
        nv.count_launch(2)
        xbuf.zero_(); fill.zero_()
        ep.barrier(dev)                                           # peers have read my outputs; everyone's input buffers are clear
        ctx.save_for_backward(dest, wc, xsave, h, pre, W1, b1, W2, b2, counts if counts is not None else torch.empty(0))
        ctx.cfg = (act, cap, ep, T, d, k, E_local, hid)
        return out

    @staticmethod
    def backward(ctx, dout):
        dest, wc, xb, h, pre, W1, b1, W2, b2, counts = ctx.saved_tensors
        counts = counts if counts.numel() else None
        act, cap, ep, T, d, k, E_local, hid = ctx.cfg
        world, rows, dev = ep.world, E_local * cap, dout.device
        lib = nv.cuda()
        ybuf, yptrs = ep.buffer("y", rows * d, torch.bfloat16, dev)
        dybuf, dyptrs = ep.buffer("dy", rows * d, torch.bfloat16, dev)
        dxbuf, dxptrs = ep.buffer("dx", rows * d, torch.bfloat16, dev)
        # the expert outputs are needed once more (d of the gate weights): recomputed from h straight into the shared buffer
        gemm(h, F.lp(W2), bias=b2.detach() if b2 is not None else None, out=ybuf.view(E_local, cap, d), m_valid=counts)
        ep.barrier(dev)
        dw = torch.empty((T, k), dtype=torch.float32, device=dev)
        dc = dout.contiguous()
        nv.check(lib.b200_moe_combine_bwd(_ptr_array(yptrs), _ptr_array(dyptrs), world, dest.data_ptr(), wc.data_ptr(), dc.data_ptr(),
                                          dw.data_ptr(), T, k, d, rows, nv.stream_ptr()), "moe_combine_bwd")
        ep.barrier(dev)
        dy = dybuf.view(E_local, cap, d)
        W1l, W2l = F.lp(W1), F.lp(W2)
        dh = gemm(dy, W2l, b_mn=True, aux_in=pre, dact=act, m_valid=counts)                   # [E, cap, hid]
        dW2 = gemm(dy, h, a_mn=True, b_mn=True, out_dtype=torch.float32, k_valid=counts)       # [E, d, hid]
        dW1 = gemm(dh, xb, a_mn=True, b_mn=True, out_dtype=torch.float32, k_valid=counts)      # [E, hid, d]
        gemm(dh, W1l, b_mn=True, out=dxbuf.view(E_local, cap, d), m_valid=counts)               # [E, cap, d], pulled by the token owners
        db1 = db2 = None
        if b1 is not None:
            db1 = torch.zeros((E_local, hid), dtype=torch.float32, device=dev)
            nv.check(lib.b200_colsum_batched(dh.data_ptr(), db1.data_ptr(), E_local, cap, hid, hid, cap * hid, 1, nv.ptr(counts), nv.stream_ptr()), "colsum_batched")
        if b2 is not None:
            db2 = torch.zeros((E_local, d), dtype=torch.float32, device=dev)
            nv.check(lib.b200_colsum_batched(dy.data_ptr(), db2.data_ptr(), E_local, cap, d, d, cap * d, 1, nv.ptr(counts), nv.stream_ptr()), "colsum_batched")
        # adjoint of dispatch: pull the token gradients back from the owning ranks
        ep.barrier(dev)
        dx = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
        nv.check(lib.b200_moe_gather_sum(_ptr_array(dxptrs), world, dest.data_ptr(), dx.data_ptr(), T, k, d, rows, nv.stream_ptr()), "moe_gather_sum")
        nv.count_launch(4)
        dybuf.zero_()
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
                 shared_hidden=0, num_shared=0, ep_group=None, ep_backend="fused"):
        self.d_in, self.E, self.top_k, self.act, self.routing = d_in, num_experts, min(top_k, num_experts), act, routing
        self.capacity_factor, self.aux_coef, self.renorm = capacity_factor, aux_coef, renorm
        self.gate = nn.Linear(d_in, num_experts, init=init)
        self.shared = [_Expert(d_in, shared_hidden, act, init) for _ in range(num_shared)]
        self.ep = EPContext(ep_group, backend=ep_backend) if ep_group is not None else None
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
        if self.ep is not None and world > 1:
            for p in (self.W1, self.b1, self.W2, self.b2):
                p._ep_sharded = True            # owned by this rank alone: no gradient reduction across the group
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
        if self.ep is not None and self.ep.world > 1 and (not x2.is_cuda or self.ep.backend == "nccl"):
            routed = _experts_all_to_all(x2, idx, w, self.W1, self.b1, self.W2, self.b2, self.act, self.ep)
        elif x2.is_cuda and x2.dtype == torch.bfloat16:
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


class _AllToAllFn(Function):
    """Differentiable `all_to_all_single` over rows: the backward is the same exchange with the split lists swapped."""

    @staticmethod
    def forward(ctx, x, send, recv, group):
        import torch.distributed as dist
        ctx.cfg = (send, recv, group)
        out = torch.empty((sum(recv),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        send, recv, group = ctx.cfg
        out = torch.empty((sum(send),) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=send, input_split_sizes=recv, group=group)
        return out, None, None, None


def _experts_all_to_all(x, idx, w, W1, b1, W2, b2, act, ep: "EPContext"):
    """Expert parallelism the library way: sort the (token, choice) pairs by expert, exchange counts, all-to-all the
    rows to the ranks that own their experts, run each local expert on its rows, all-to-all back, weight and sum.
    No capacity limit (no drops). This is the baseline the peer-memory kernels are measured against (NCCL on GPUs) and
    the path CPU (gloo) ranks take; the split sizes are read on the host, so it cannot be captured in a CUDA graph."""
    import torch.distributed as dist
    T, d = x.shape
    k = idx.shape[1]
    E_local, world = W1.shape[0], ep.world
    flat_e = idx.reshape(-1).long()
    order = torch.argsort(flat_e, stable=True)                     # pairs grouped by global expert id (= by owner rank)
    tok = torch.div(order, k, rounding_mode="floor")
    counts = torch.bincount(flat_e, minlength=E_local * world)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=ep.group)    # [src rank][local expert]
    send = counts.view(world, E_local).sum(1).tolist()
    rc = recv_counts.view(world, E_local)
    recv = rc.sum(1).tolist()
    rows = _AllToAllFn.apply(x[tok], send, recv, ep.group)         # grouped by source rank, then by local expert
    # regroup by local expert
    src_e = torch.repeat_interleave(torch.arange(world * E_local, device=x.device) % E_local, rc.reshape(-1))
    by_e = torch.argsort(src_e, stable=True)
    rows_e = rows[by_e]
    per_e = rc.sum(0).tolist()
    outs, off = [], 0
    for e in range(E_local):
        seg = rows_e[off:off + per_e[e]]
        off += per_e[e]
        if seg.shape[0] == 0:
            outs.append(seg.new_zeros((0, d)))
            continue
        hcur = F.linear(seg, W1[e], b1[e] if b1 is not None else None, act, None)
        outs.append(F.linear(hcur, W2[e], b2[e] if b2 is not None else None, "none", None))
    y_e = torch.cat(outs, 0) if outs else rows_e
    y_src = torch.empty_like(y_e).index_copy(0, by_e, y_e) if y_e.shape[0] else y_e
    back = _AllToAllFn.apply(y_src, recv, send, ep.group)          # in `order` again
    contrib = back.float() * w.reshape(-1)[order].float().unsqueeze(1)
    out = torch.zeros((T, d), dtype=torch.float32, device=x.device).index_add(0, tok, contrib)
    return out.to(x.dtype)


def F_add(a, b):
    from .looped_transformer import _add
    return _add(a, b)


class NormalMoE(_RoutedMoE):
    """`NormalMoE::new(in, hidden, E)` (src/nn.rs:397-434): gate Linear(in, E), experts Linear -> ReLU -> Linear."""

    def __init__(self, in_features: int, hidden_features: int, num_experts: int, top_k: int = 2, routing: str = "topk",
                 act: str = "relu", capacity_factor: float = 1.5, aux_coef: float = 0.01, renorm: bool = True,
                 init=nn.he_normal, ep_group=None, ep_backend="fused"):
        super().__init__(in_features, hidden_features, num_experts, top_k, act, routing, capacity_factor, aux_coef, renorm, init,
                         ep_group=ep_group, ep_backend=ep_backend)


class FineGrainedMoE(_RoutedMoE):
    """`FineGrainedMoE::new(in, shared_hidden, expert_hidden, E)` (src/nn.rs:445-496): gate, one shared expert
    (`num_shared` generalises it), E small routed experts."""

    def __init__(self, in_features: int, shared_hidden: int, expert_hidden: int, num_experts: int, top_k: int = 6,
                 num_shared: int = 1, routing: str = "topk", act: str = "relu", capacity_factor: float = 1.25,
                 aux_coef: float = 0.01, renorm: bool = True, init=nn.he_normal, ep_group=None, ep_backend="fused"):
        super().__init__(in_features, expert_hidden, num_experts, top_k, act, routing, capacity_factor, aux_coef, renorm, init,
                         shared_hidden=shared_hidden, num_shared=num_shared, ep_group=ep_group, ep_backend=ep_backend)


class MoETransformerLM(nn.Module):
    """Token embedding -> L x (LN -> causal MHA -> residual; LN -> FineGrainedMoE -> residual) -> LN -> LM head.
    The loss adds the routers' load-balance terms."""

    def __init__(self, vocab: int, d_model: int, layers: int, heads: int, num_experts: int, top_k: int, num_shared: int,
                 expert_hidden: int, max_seq: int, init_std: float = 0.02, ep_group=None, act: str = "silu",
                 capacity_factor: float = 1.25, ep_backend: str = "fused"):
        from .looped_transformer import MultiHeadAttention
        init = nn.normal_init(init_std)
        self.tok = nn.Embedding(vocab, d_model, std=init_std)
        self.pos = nn.Embedding(max_seq, d_model, std=init_std)
        self.ln1 = [nn.LayerNorm(d_model) for _ in range(layers)]
        self.attn = [MultiHeadAttention(d_model, heads, causal=True, init=init) for _ in range(layers)]
        self.ln2 = [nn.LayerNorm(d_model) for _ in range(layers)]
        self.ep_group = ep_group
        self.moe = [FineGrainedMoE(d_model, expert_hidden, expert_hidden, num_experts, top_k=top_k, num_shared=num_shared, act=act,
                                   init=init, ep_group=ep_group, capacity_factor=capacity_factor, ep_backend=ep_backend) for _ in range(layers)]
        # one set of dispatch / combine buffers for all layers (they are used one layer at a time)
        for m in self.moe[1:]:
            if m.ep is not None:
                m.ep = self.moe[0].ep
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

    def make_optimizer(self, lr: float = 1e-3, mode: str = "fused", **kw):
        """The optimizer that matches this model's parallel layout: under expert parallelism every rank trains on its own
        batch, so the shared parameters (attention, routers, shared experts, embeddings, norms, head) are data-parallel
        (`DistributedAdam`, gradients averaged) while each routed expert lives on one rank, whose local Adam scales the
        summed contributions of all ranks' losses by 1/world."""
        import torch.distributed as dist
        from ..optim import Adam, MultiOptimizer
        world = dist.get_world_size(self.ep_group) if self.ep_group is not None else 1
        if world == 1:
            return Adam(self.parameters(), lr=lr, **kw)
        from ..parallel.ddp import DistributedAdam
        owned = [p for p in self.parameters() if getattr(p, "_ep_sharded", False)]
        shared = [p for p in self.parameters() if not getattr(p, "_ep_sharded", False)]
        local = Adam(owned, lr=lr, **kw)
        local.grad_scale = torch.full((1,), 1.0 / world, dtype=torch.float32, device=owned[0].device)
        return MultiOptimizer([DistributedAdam(shared, lr=lr, group=self.ep_group, mode=mode, **kw), local])

    def loss(self, ids, labels):
        from ..ops.transformer import lm_head_ce
        h, aux = self.hidden(ids)
        l = lm_head_ce(h, self.lm_head.weight, None, labels)
        return l if aux is None else l + aux.to(l.dtype)

    def forward(self, ids):
        return self.lm_head(self.hidden(ids)[0])


class _ExpertView(nn.Module):
    """Expert `e` of a routed layer on its own: `forward(x) = act(x W1[e]^T + b1[e]) W2[e]^T + b2[e]` on views of the
    layer's stacked expert weights (the reference keeps a `Vec<Sequential>`, src/nn.rs:391-394; here the experts are
    rows of four stacked tensors so that one grouped GEMM serves them all)."""

    def __init__(self, moe, e: int):
        self._moe, self.index = moe, e

    def parameters(self):
        m, e = self._moe, self.index
        return [m.W1[e], m.b1[e], m.W2[e], m.b2[e]]

    def forward(self, x):
        from ..ops.gemm import act_ref
        w1, b1, w2, b2 = self.parameters()
        h = act_ref(x.float() @ w1.float().t() + b1.float(), self._moe.act)
        return (h @ w2.float().t() + b2.float()).to(x.dtype)


from .._compat import alias_fields as _alias_fields  # noqa: E402

_alias_fields(_RoutedMoE, experts=lambda self: [_ExpertView(self, e) for e in range(self.W1.shape[0])],
              shared_expert=lambda self: self.shared[0] if len(self.shared) == 1 else (self.shared or None))
