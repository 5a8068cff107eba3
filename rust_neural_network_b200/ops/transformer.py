"""Fused pre-norm transformer block and fused LM-head + cross-entropy, forward and backward written
out by hand as sequences of this package's kernels (no autograd graph inside the block).

Block math (rust-nn src/looped_transformer.rs:150-202): h = x + Attn(LN1 x); out = h + FF(LN2 h),
FF = Linear -> GELU -> Linear, Attn = out_proj(softmax(q k^T/sqrt(hd)) v) with q,k,v from three
biased Linears (src/looped_transformer.rs:59-143). Per block the forward is 7 launches:
LN, fused QKV GEMM (+bias), flash attention on strided views of the QKV buffer (no head
split/merge copies), out-proj GEMM (+bias +residual), LN, FF1 GEMM (+bias, GELU, pre-activation kept),
FF2 GEMM (+bias +residual). The backward fuses the GELU derivative into the dX GEMM epilogue, the
residual gradients into the LayerNorm backward, and accumulates weight gradients straight into
the optimizer's flat fp32 gradient buffer.
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

from . import kernels as K
from .functional import _bgrad, _scale_by, _wgrad, lp
from .gemm import gemm


def _adjacent(a, b, c):
    """True when a, b, c are contiguous tensors laid out back to back inside ONE storage."""
    es = a.element_size()
    sa = a.untyped_storage()
    if not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        return False
    if b.untyped_storage().data_ptr() != sa.data_ptr() or c.untyped_storage().data_ptr() != sa.data_ptr():
        return False
    return b.data_ptr() == a.data_ptr() + a.numel() * es and c.data_ptr() == b.data_ptr() + b.numel() * es


def _fused_qkv(wq, wk, wv, getter):
    """[3d, d] matrix holding q, k, v weights (zero-copy when they are adjacent in one storage)."""
    a, b, c = getter(wq), getter(wk), getter(wv)
    if _adjacent(a, b, c):
        return torch.as_strided(a, (a.shape[0] * 3, a.shape[1]), (a.shape[1], 1))
    return torch.cat([a, b, c], 0)


def _fused_vec(bq, bk, bv, getter):
    a, b, c = getter(bq), getter(bk), getter(bv)
    if _adjacent(a, b, c):
        return torch.as_strided(a, (a.numel() * 3,), (1,))
    return torch.cat([a, b, c], 0)


class TransformerBlockFn(Function):
    """x [B, S, d] bf16 -> [B, S, d] bf16."""

    @staticmethod
    def forward(ctx, x, g1, be1, wq, bq, wk, bk, wv, bv, wo, bo, g2, be2, w1, b1, w2, b2, heads, causal, eps):
        B, S, d = x.shape
        T = B * S
        hd = d // heads
        x2 = x.reshape(T, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        h1, mean1, rstd1 = K.layernorm_fwd(x2, g1.detach(), be1.detach(), eps)
        wqkv = _fused_qkv(wq, wk, wv, lp)
        bqkv = _fused_vec(bq, bk, bv, lambda t: t.detach())
        qkv = gemm(h1, wqkv, bias=bqkv)                                   # [T, 3d]
        qkv5 = qkv.view(B, S, 3, heads, hd)
        o, lse = K.flash_fwd(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], 1.0 / math.sqrt(hd), causal)
        o2 = o.view(T, d)
        # x + attn and its LayerNorm in one pass: the add is cheaper here than in the projection's epilogue
        y1, h2, mean2, rstd2 = K.add_layernorm_fwd(gemm(o2, lp(wo), bias=bo.detach()), x2, g2.detach(), be2.detach(), eps)
        a, pre = gemm(h2, lp(w1), bias=b1.detach(), act="gelu", want_aux=True)
        y2 = gemm(a, lp(w2), bias=b2.detach(), residual=y1)               # h + ff
        ctx.save_for_backward(x2, mean1, rstd1, h1, qkv, o, lse, y1, mean2, rstd2, h2, pre, a,
                              g1, be1, wq, bq, wk, bk, wv, bv, wo, bo, g2, be2, w1, b1, w2, b2)
        ctx.cfg = (B, S, d, heads, causal)
        return y2.view(B, S, d)

    @staticmethod
    def backward(ctx, dy):
        (x2, mean1, rstd1, h1, qkv, o, lse, y1, mean2, rstd2, h2, pre, a,
         g1, be1, wq, bq, wk, bk, wv, bv, wo, bo, g2, be2, w1, b1, w2, b2) = ctx.saved_tensors
        B, S, d, heads, causal = ctx.cfg
        T, hd = B * S, d // heads
        dy2 = dy.reshape(T, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # ---- feed-forward
        dw2 = _wgrad(dy2, a, w2)
        # the bias gradients of the two projections that feed the residual stream around the second LayerNorm (ff2: column
        # sums of dy2; out-projection: column sums of what that LayerNorm's backward returns) come out of its backward pass
        acc_b2 = b2.grad if (getattr(b2, "_fused_grad", False) and b2.grad is not None) else torch.zeros(d, dtype=torch.float32, device=dy2.device)
        acc_bo = bo.grad if (getattr(bo, "_fused_grad", False) and bo.grad is not None) else torch.zeros(d, dtype=torch.float32, device=dy2.device)
        # (dy W2) * gelu'(pre): the product is a plain GEMM, the derivative and the bias gradient are one streaming pass
        fused_b1 = getattr(b1, "_fused_grad", False) and b1.grad is not None
        dpre, db1 = K.dact_colsum(gemm(dy2, lp(w2), b_mn=True), pre, "gelu", bias_grad=b1.grad if fused_b1 else None)
        dw1 = _wgrad(dpre, h2, w1)
        dh2 = gemm(dpre, lp(w1), b_mn=True)
        fused_ln2 = getattr(g2, "_fused_grad", False) and g2.grad is not None
        dy1, dg2, dbe2 = K.layernorm_bwd(dh2, y1, g2.detach(), mean2, rstd2, dres=dy2,
                                         dgamma=g2.grad if fused_ln2 else None, dbeta=be2.grad if fused_ln2 else None,
                                         sum_dres=acc_b2, sum_dx=acc_bo)
        db2 = None if acc_b2 is b2.grad else acc_b2
        dbo = None if acc_bo is bo.grad else acc_bo
        # ---- attention
        o2 = o.view(T, d)
        dwo = _wgrad(dy1, o2, wo)
        do = gemm(dy1, lp(wo), b_mn=True).view(B, S, heads, hd)
        dqkv = torch.empty_like(qkv)
        qkv5, dqkv5 = qkv.view(B, S, 3, heads, hd), dqkv.view(B, S, 3, heads, hd)
        K.flash_bwd(do, qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], o, lse, 1.0 / math.sqrt(hd), causal,
                    dq=dqkv5[:, :, 0], dk=dqkv5[:, :, 1], dv=dqkv5[:, :, 2])
        # weight / bias gradients of the fused QKV projection
        fused_w = all(getattr(t, "_fused_grad", False) and t.grad is not None for t in (wq, wk, wv))
        if fused_w:
            gw = _fused_qkv(wq, wk, wv, lambda t: t.grad)
            if gw.data_ptr() == wq.grad.data_ptr():
                gemm(dqkv, h1, a_mn=True, b_mn=True, accumulate_into=gw)
                dwq = dwk = dwv = None
            else:
                fused_w = False
        if not fused_w:
            dwqkv = gemm(dqkv, h1, a_mn=True, b_mn=True, out_dtype=torch.float32)
            dwq, dwk, dwv = dwqkv[:d], dwqkv[d:2 * d], dwqkv[2 * d:]
        fused_b = all(getattr(t, "_fused_grad", False) and t.grad is not None for t in (bq, bk, bv))
        if fused_b:
            gb = _fused_vec(bq, bk, bv, lambda t: t.grad)
            if gb.data_ptr() == bq.grad.data_ptr():                     # adjacent in the flat gradient buffer: accumulate in place
                K.colsum(dqkv, out=gb)
                dbq = dbk = dbv = None
            else:
                fused_b = False
        if not fused_b:
            dbqkv = K.colsum(dqkv)
            dbq, dbk, dbv = dbqkv[:d], dbqkv[d:2 * d], dbqkv[2 * d:]
        dh1 = gemm(dqkv, _fused_qkv(wq, wk, wv, lp), b_mn=True)
        fused_ln1 = getattr(g1, "_fused_grad", False) and g1.grad is not None
        dx, dg1, dbe1 = K.layernorm_bwd(dh1, x2, g1.detach(), mean1, rstd1, dres=dy1,
                                        dgamma=g1.grad if fused_ln1 else None, dbeta=be1.grad if fused_ln1 else None)
        if fused_ln1: dg1 = dbe1 = None
        if fused_ln2: dg2 = dbe2 = None
        return (dx.view(B, S, d), dg1, dbe1, dwq, dbq, dwk, dbk, dwv, dbv, dwo, dbo, dg2, dbe2, dw1, db1, dw2, db2,
                None, None, None)


def transformer_block(x, blk, causal):
    """Run `blk` (a `models.looped_transformer.TransformerBlock`) through the fused function."""
    at = blk.attn
    return TransformerBlockFn.apply(
        x, blk.ln1.gamma, blk.ln1.beta, at.q_proj.weight, at.q_proj.bias, at.k_proj.weight, at.k_proj.bias,
        at.v_proj.weight, at.v_proj.bias, at.out_proj.weight, at.out_proj.bias, blk.ln2.gamma, blk.ln2.beta,
        blk.ff1.weight, blk.ff1.bias, blk.ff2.weight, blk.ff2.bias, at.heads, causal, blk.ln1.eps)


class LMHeadCEFn(Function):
    """mean CE(h W^T + b, labels): logits GEMM, then one kernel that produces the loss and overwrites
    the logits with d(loss)/d(logits); backward is two GEMMs and a column sum."""

    @staticmethod
    def forward(ctx, h, w, b, labels):
        d = h.shape[-1]
        h2 = h.reshape(-1, d)
        W = lp(w) if h2.dtype == torch.bfloat16 else w.detach()
        logits = gemm(h2, W, bias=b.detach() if b is not None else None)
        lab = labels.reshape(-1)
        if logits.is_cuda:
            from .. import _native as nv
            rows, V = logits.shape
            loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
            nv.check(nv.cuda().b200_ce_label(logits.data_ptr(), lab.contiguous().data_ptr(), logits.data_ptr(), 0,
                                             loss.data_ptr(), rows, V, logits.stride(0), 1.0 / rows, 1.0 / rows,
                                             1 if logits.dtype == torch.bfloat16 else 0, nv.stream_ptr()), "ce_label")
            nv.count_launch()
            loss, dlogits = loss.view(()), logits
        else:
            loss, dlogits = K.ce_label(logits, lab)
        ctx.save_for_backward(h2, w, b, dlogits)
        ctx.h_shape = h.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        h2, w, b, dlogits = ctx.saved_tensors
        W = lp(w) if h2.dtype == torch.bfloat16 else w.detach()
        dl = dlogits.to(h2.dtype) if dlogits.dtype != h2.dtype else dlogits
        # the saved dlogits assume an upstream gradient of 1; `g` (a device scalar) rescales inside the GEMMs
        gs = g.reshape(1).float()
        dh = gemm(dl, W, b_mn=True, alpha_t=gs)
        dw = _wgrad(dl, h2, w, alpha_t=gs)
        db = None
        if b is not None:
            db = _scale_by(K.colsum(dl), g)
            if getattr(b, "_fused_grad", False) and b.grad is not None:
                b.grad.add_(db); db = None
        return dh.view(ctx.h_shape), dw, db, None


def lm_head_ce(h, w, b, labels):
    return LMHeadCEFn.apply(h, w, b, labels)
