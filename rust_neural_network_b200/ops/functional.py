"""Differentiable ops: one ``torch.autograd.Function`` per fused op of the reference's autograd
engine (rust-nn src/tensor.rs:67-130 lists its 23 `Op` variants; the fused ones are
`linear_layer` :747, `flash_attention` :618, `layer_norm` :1013, `cross_entropy_logits` :464, ...).

PyTorch supplies the graph and the backward scheduling; every forward and backward body below is
a launch of this package's own kernels (or, for CPU tensors, the fp32 PyTorch reference).
Unlike the reference, tanh / softmax / gelu are differentiable here.
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

from . import kernels as K
from .gemm import gemm

_BWD_FROM_INPUT = {"relu": "relu_bwd", "gelu": "gelu_bwd", "silu": "silu_bwd", "sigmoid": "sigmoid_bwd",
                   "tanh": "tanh_bwd", "softplus": "softplus_bwd"}


# ----------------------------------------------------------------------------- low-precision shadows
def lp(p: torch.Tensor) -> torch.Tensor:
    """bf16 shadow of an fp32 parameter. Optimizers of this package rewrite the shadow in the same
    kernel that updates the master weight; anything else that changes the parameter in place bumps
    its version counter and triggers a re-cast here."""
    s = getattr(p, "_lp", None)
    if s is None or getattr(p, "_lp_version", -1) != p._version or s.device != p.device:
        if s is None or s.shape != p.shape or s.device != p.device:
            s = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
        s.copy_(p.detach())
        p._lp = s
        p._lp_version = p._version
    return s


def compute_weight(w: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    if like.dtype == torch.bfloat16:
        return lp(w)
    if getattr(w, "_dp_sharded", False):
        raise RuntimeError("fp32 compute reads the fp32 master weights, which a sharded data-parallel optimizer keeps "
                           "current only on the owning rank: use bf16 compute, or DistributedAdam(mode='nccl')")
    return w.detach()


def _wgrad(g2, x2, w, alpha_t=None):
    """dW = g^T x (times the optional device scalar `alpha_t`). If the parameter carries a pre-set
    fp32 `.grad` owned by a flat optimizer buffer (`_fused_grad`), accumulate straight into it and
    return None so autograd adds nothing."""
    if getattr(w, "_fused_grad", False) and w.grad is not None:
        gemm(g2, x2, a_mn=True, b_mn=True, accumulate_into=w.grad, alpha_t=alpha_t)
        return None
    return gemm(g2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32, alpha_t=alpha_t)


def _bgrad(g2, b):
    if b is None:
        return None
    if getattr(b, "_fused_grad", False) and b.grad is not None:
        K.colsum(g2, out=b.grad)
        return None
    return K.colsum(g2)


# ----------------------------------------------------------------------------- linear
class LinearFn(Function):
    """y = act(x W^T + b) (+ residual); x [..., in], W [out, in]."""

    @staticmethod
    def forward(ctx, x, w, b, act, residual):
        in_f = w.shape[1]
        x2 = x.reshape(-1, in_f)
        W = compute_weight(w, x2)
        bias = b.detach() if b is not None else None
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        if act == "none":
            y = gemm(x2, W, bias=bias, residual=res2); saved = None; mode = None
        elif act in ("gelu", "silu") or res2 is not None:
            # keep the pre-activation: the derivative is evaluated from it in backward
            y, saved = gemm(x2, W, bias=bias, act=act, residual=res2, want_aux=True)
            mode = act + "_bwd"
        else:
            y = gemm(x2, W, bias=bias, act=act); saved = y
            mode = {"relu": "relu_bwd", "sigmoid": "sigmoid_bwd_out", "tanh": "tanh_bwd_out"}[act]
        ctx.save_for_backward(x2, w, b, saved)
        ctx.mode = mode
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        ctx.res_shape = residual.shape if residual is not None else None
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, b, saved = ctx.saved_tensors
        g = dy.reshape(-1, w.shape[0])
        if not g.is_contiguous():
            g = g.contiguous()
        g0 = g
        if ctx.mode is not None:
            g = K.binary(g, saved, ctx.mode)
        W = compute_weight(w, x2)
        g = g.to(x2.dtype) if g.dtype != x2.dtype else g
        dx = gemm(g, W, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad(g, x2, w) if ctx.needs_input_grad[1] else None
        db = _bgrad(g, b) if (b is not None and ctx.needs_input_grad[2]) else None
        dres = g0.view(ctx.res_shape) if (ctx.has_res and ctx.needs_input_grad[4]) else None
        return dx, dw, db, None, dres


def linear(x, w, b=None, act="none", residual=None):
    return LinearFn.apply(x, w, b, act, residual)


# ----------------------------------------------------------------------------- matmul (2-D or batched)
def _mm(a, b, out_dtype=None):
    """a [.., M, K] @ b [.., K, N] where either operand may be a transposed VIEW: the view's layout
    becomes the kernel's K-major / MN-major flag, so no transposed copy is made."""
    if a.stride(-1) == 1:
        A, a_mn = a, False
    elif a.stride(-2) == 1:
        A, a_mn = a.transpose(-1, -2), True            # stored [K, M]
    else:
        A, a_mn = a.contiguous(), False
    if b.stride(-1) == 1:
        Bm, b_mn = b, True                             # stored [K, N]
    elif b.stride(-2) == 1:
        Bm, b_mn = b.transpose(-1, -2), False          # stored [N, K]
    else:
        Bm, b_mn = b.contiguous(), True
    if A.dtype != Bm.dtype:
        Bm = Bm.to(A.dtype)
    return gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out_dtype=out_dtype)


class MatmulFn(Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return _mm(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        if g.stride(-1) != 1 and g.stride(-2) != 1:
            g = g.contiguous()
        g = g.to(a.dtype) if g.dtype != a.dtype else g
        da = _mm(g, b.transpose(-1, -2)) if ctx.needs_input_grad[0] else None       # g @ b^T
        db = _mm(a.transpose(-1, -2), g) if ctx.needs_input_grad[1] else None       # a^T @ g
        return da, db


def matmul(a, b):
    """a [.., M, K] @ b [.., K, N] on the tcgen05 GEMM."""
    return MatmulFn.apply(a, b)


# ----------------------------------------------------------------------------- elementwise
class UnaryFn(Function):
    @staticmethod
    def forward(ctx, x, op):
        ctx.save_for_backward(x)
        ctx.op = op
        return K.unary(x, op)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return K.binary(g.contiguous().to(x.dtype), x, _BWD_FROM_INPUT[ctx.op]), None


def relu(x): return UnaryFn.apply(x, "relu")
def gelu(x): return UnaryFn.apply(x, "gelu")
def silu(x): return UnaryFn.apply(x, "silu")
def sigmoid(x): return UnaryFn.apply(x, "sigmoid")
def tanh(x): return UnaryFn.apply(x, "tanh")
def softplus(x): return UnaryFn.apply(x, "softplus")


class MulSiluFn(Function):
    """y * silu(z): the Mamba output gate (rust-nn src/mamba.rs:108-110) as one kernel."""

    @staticmethod
    def forward(ctx, y, z):
        ctx.save_for_backward(y, z)
        return K.gate_fwd(y, z)

    @staticmethod
    def backward(ctx, g):
        y, z = ctx.saved_tensors
        return K.gate_bwd(g, y, z)


def mul_silu(y, z): return MulSiluFn.apply(y, z)


class DropoutFn(Function):
    @staticmethod
    def forward(ctx, x, p, seed):
        ctx.p, ctx.seed = p, seed
        return K.dropout_mask_apply(x, p, seed)

    @staticmethod
    def backward(ctx, g):
        return K.dropout_mask_apply(g.contiguous(), ctx.p, ctx.seed), None, None


def dropout(x, p, seed): return DropoutFn.apply(x, p, seed)


class FakeQuantFn(Function):
    """clamp(round(x/s), qmin, qmax) * s with a straight-through gradient inside the clamp range
    (the reference documents STE but detaches the output, rust-nn src/nn.rs:657-667)."""

    @staticmethod
    def forward(ctx, x, scale, qmin, qmax):
        ctx.save_for_backward(x)
        ctx.lo, ctx.hi = qmin * scale, qmax * scale
        return K.fake_quant(x, scale, qmin, qmax)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        mask = ((x >= ctx.lo) & (x <= ctx.hi)).to(g.dtype)
        return g * mask, None, None, None


def fake_quantize(x, scale, qmin, qmax): return FakeQuantFn.apply(x, scale, qmin, qmax)


# ----------------------------------------------------------------------------- softmax
class SoftmaxFn(Function):
    """softmax(scale * x) over the last axis, optionally with the causal mask of [.., S, S] score matrices."""

    @staticmethod
    def forward(ctx, x, scale, causal_period):
        y = K.softmax_fwd(x, scale, causal_period)
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return K.softmax_bwd(g, y, ctx.scale), None, None


def softmax(x, scale: float = 1.0, causal_period: int = 0): return SoftmaxFn.apply(x, float(scale), int(causal_period))


# ----------------------------------------------------------------------------- embedding
class EmbeddingFn(Function):
    @staticmethod
    def forward(ctx, ids, table, out_dtype):
        T = lp(table) if out_dtype == torch.bfloat16 else table.detach()
        ctx.save_for_backward(ids, table)
        return K.embedding_fwd(T, ids)

    @staticmethod
    def backward(ctx, g):
        ids, table = ctx.saved_tensors
        g = g.contiguous()
        if getattr(table, "_fused_grad", False) and table.grad is not None and table.is_cuda:
            from .. import _native as nv
            ids_c = ids.contiguous().view(-1)
            nv.check(nv.cuda().b200_embedding_bwd(g.data_ptr(), ids_c.data_ptr(), table.grad.data_ptr(), ids_c.numel(),
                                                  table.shape[1], table.shape[0], 1 if g.dtype == torch.bfloat16 else 0,
                                                  nv.stream_ptr()), "embedding_bwd")
            nv.count_launch()
            return None, None, None
        return None, K.embedding_bwd(g, ids, table.shape[0]), None


def embedding(ids, table, out_dtype=torch.float32): return EmbeddingFn.apply(ids, table, out_dtype)


# ----------------------------------------------------------------------------- normalisation
class LayerNormFn(Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        y, mean, rstd = K.layernorm_fwd(x2, gamma.detach(), beta.detach(), eps)
        ctx.save_for_backward(x2, gamma, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, gamma, mean, rstd = ctx.saved_tensors
        dx, dg, db = K.layernorm_bwd(dy.reshape(x2.shape).to(x2.dtype), x2, gamma.detach(), mean, rstd)
        return dx.view(ctx.shape), dg, db, None


def layer_norm(x, gamma, beta, eps=1e-5): return LayerNormFn.apply(x, gamma, beta, eps)


class BatchNormFn(Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, run_mean, run_var, eps, momentum, training):
        y, mean, rstd = K.batchnorm_fwd(x, gamma.detach(), beta.detach(), run_mean, run_var, eps, momentum, training)
        ctx.save_for_backward(x, gamma, mean, rstd)
        ctx.training = training
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        dx, dg, db = K.batchnorm_bwd(dy.contiguous().to(x.dtype), x, gamma.detach(), mean, rstd, ctx.training)
        return dx, dg, db, None, None, None, None, None


def batch_norm(x, gamma, beta, run_mean, run_var, eps, momentum, training):
    return BatchNormFn.apply(x, gamma, beta, run_mean, run_var, eps, momentum, training)


# ----------------------------------------------------------------------------- losses
def _scale_by(grad, g):
    """grad * g where g is the 0-d upstream gradient (no host sync)."""
    if g is None:
        return grad
    return K.binary(grad, g.reshape(1).to(grad.dtype), "mul") if grad.is_cuda else grad * g.to(grad.dtype)


class CrossEntropyLabelFn(Function):
    @staticmethod
    def forward(ctx, logits, labels):
        V = logits.shape[-1]
        loss, grad = K.ce_label(logits.reshape(-1, V), labels.reshape(-1), want_grad=logits.requires_grad)
        ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return _scale_by(grad, g).view(ctx.shape), None


class CrossEntropyDenseFn(Function):
    @staticmethod
    def forward(ctx, logits, target):
        V = logits.shape[-1]
        loss, grad = K.ce_dense(logits.reshape(-1, V), target.reshape(-1, V), want_grad=logits.requires_grad)
        ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return _scale_by(grad, g).view(ctx.shape), None


def cross_entropy(logits, target):
    """Mean cross-entropy. `target` is either integer class ids or a dense one-hot / soft target
    of the logits' shape (the reference's only form, rust-nn src/tensor.rs:464-496)."""
    if target.dtype in (torch.int64, torch.int32):
        return CrossEntropyLabelFn.apply(logits, target.long())
    return CrossEntropyDenseFn.apply(logits, target)


class PointwiseLossFn(Function):
    @staticmethod
    def forward(ctx, pred, target, kind, delta, reduction):
        loss, grad = K.pointwise_loss(pred, target, kind, delta, reduction, want_grad=pred.requires_grad)
        ctx.save_for_backward(grad)
        ctx.shape = pred.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return _scale_by(grad, g).view(ctx.shape), None, None, None, None


def pointwise_loss(pred, target, kind, delta=1.0, reduction="mean"):
    return PointwiseLossFn.apply(pred, target, kind, delta, reduction)


# ----------------------------------------------------------------------------- attention
class FlashAttnFn(Function):
    """softmax(q k^T * scale) v on [B, S, H, hd] views (strided views of a fused QKV buffer are fine)."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal):
        in_dtype = q.dtype
        if q.is_cuda and in_dtype != torch.bfloat16:
            q, k, v = (K.cast(t.contiguous(), torch.bfloat16) for t in (q, k, v))
        o, lse = K.flash_fwd(q, k, v, scale, causal)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.causal, ctx.in_dtype = scale, causal, in_dtype
        return o.to(in_dtype) if o.dtype != in_dtype else o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        if not q.is_cuda:
            with torch.enable_grad():
                qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
                ref = K.attention_ref(qr, kr, vr, ctx.scale, ctx.causal)
                gq, gk, gv = torch.autograd.grad(ref, (qr, kr, vr), do.float())
            return gq.to(ctx.in_dtype), gk.to(ctx.in_dtype), gv.to(ctx.in_dtype), None, None
        if do.dtype != torch.bfloat16:
            do = K.cast(do.contiguous(), torch.bfloat16)
        dq, dk, dv = K.flash_bwd(do, q, k, v, o, lse, ctx.scale, ctx.causal)
        if ctx.in_dtype != torch.bfloat16:
            dq, dk, dv = (K.cast(t, ctx.in_dtype) for t in (dq, dk, dv))
        return dq, dk, dv, None, None


def flash_attention(q, k, v, scale=None, causal=False):
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return FlashAttnFn.apply(q, k, v, float(scale), bool(causal))
