"""Linear attention (rust-nn src/linear_attention.rs): feature maps phi = ELU+1 or ReLU^2,
causal and non-causal, forward and backward.

    out_t = phi(s q_t) . S_t / (phi(s q_t) . z_t + eps),   S_t = sum_{u<=t} phi(s k_u) (x) v_u,  z_t = sum_{u<=t} phi(s k_u)

(non-causal: the sums run over the whole sequence). The reference computes the causal form as a
per-token rank-1 recurrence and its backward stores all seq*d^2 states (src/linear_attention.rs:214-266,
502-632). Here the causal form is CHUNKED: tokens are grouped into chunks of C; inside a chunk the
masked C x C product (phi Q)(phi K)^T is applied to [V | 1] (the extra ones column yields the
denominator for free), between chunks a d x (d+8) state is carried by an exclusive prefix sum. Every
product is a batched call of the tcgen05 GEMM kernel (NT for (phi Q)(phi K)^T, TN for the chunk states,
NN for applying them); the feature maps and the mask are this package's elementwise kernels. The
backward is the autograd composition of the same kernels (each GEMM's backward is two more GEMMs).

Inputs are [B, S, H, d] (any strides); output [B, S, H, d].
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

from . import kernels as K
from .functional import matmul

CHUNK = 128


class _PhiFn(Function):
    """phi(scale * x) with phi = elu+1 | relu^2."""

    @staticmethod
    def forward(ctx, x, scale, kind):
        xs = K.unary(x, "scale", scale) if scale != 1.0 else x.contiguous()
        ctx.save_for_backward(xs)
        ctx.scale, ctx.kind = scale, kind
        return K.unary(xs, "elu1" if kind == "elu" else "relu2", 1.0)

    @staticmethod
    def backward(ctx, g):
        (xs,) = ctx.saved_tensors
        d = K.binary(g.contiguous().to(xs.dtype), xs, "elu1_bwd" if ctx.kind == "elu" else "relu2_bwd")
        if ctx.scale != 1.0:
            d = K.unary(d, "scale", ctx.scale)
        return d, None, None


class _MulConstFn(Function):
    """x * c for a constant (non-differentiated) tensor c broadcast over the leading dims."""

    @staticmethod
    def forward(ctx, x, c):
        ctx.save_for_backward(c)
        return K.binary(x, c.to(x.dtype), "mul")

    @staticmethod
    def backward(ctx, g):
        (c,) = ctx.saved_tensors
        return K.binary(g.contiguous(), c.to(g.dtype), "mul"), None


class _DivFn(Function):
    """num / den with den broadcast over the last dim: num [.., d], den [.., 1]."""

    @staticmethod
    def forward(ctx, num, den):
        out = num / den
        ctx.save_for_backward(out, den)
        return out

    @staticmethod
    def backward(ctx, g):
        out, den = ctx.saved_tensors
        gn = g / den
        gd = -(gn * out).sum(-1, keepdim=True)
        return gn, gd


def phi(x, scale: float, kind: str):
    return _PhiFn.apply(x, float(scale), kind)


def _heads_first(t):
    """[B, S, H, d] -> contiguous [B*H, S, d]."""
    B, S, H, d = t.shape
    return t.permute(0, 2, 1, 3).reshape(B * H, S, d)


def linear_attention(q, k, v, scale: float = 1.0, eps: float = 1e-6, causal: bool = False, kind: str = "elu", chunk: int = CHUNK, sp=None):
    """[B, S, H, d] tensors. `sp`: a `parallel.sp.SPContext` when S is this rank's contiguous slice of a longer
    sequence - the KV states of the other ranks then enter through one state exchange."""
    B, S, H, d = q.shape
    dtype = q.dtype
    pq = _heads_first(phi(q, scale, kind))                  # [BH, S, d]
    pk = _heads_first(phi(k, scale, kind))
    vh = _heads_first(v)
    BH = B * H
    # [V | 1 | 0...]: the ones column carries the normaliser through the same GEMMs (width d+8 keeps 16-byte rows)
    ones = torch.zeros(BH, S, 8, dtype=dtype, device=q.device)
    ones[..., 0] = 1
    v1 = torch.cat([vh, ones], -1)                           # [BH, S, d+8]
    if not causal:
        state = matmul(pk.transpose(1, 2), v1)               # [BH, d, d+8]   (TN GEMM, K = S)
        if sp is not None:
            state = sp.all_sum(state.float()).to(dtype)      # every rank's tokens attend to every rank's state
        nd = matmul(pq, state)                               # [BH, S, d+8]
    else:
        C = min(chunk, S)
        pad = (C - S % C) % C
        if pad:
            z = lambda t: torch.cat([t, torch.zeros(BH, pad, t.shape[-1], dtype=t.dtype, device=t.device)], 1)
            pq, pk, v1 = z(pq), z(pk), z(v1)
        Sp = S + pad
        n = Sp // C
        pqc = pq.reshape(BH * n, C, d); pkc = pk.reshape(BH * n, C, d); v1c = v1.reshape(BH * n, C, d + 8)
        # inside a chunk: masked (phi Q)(phi K)^T applied to [V | 1]
        a = matmul(pqc, pkc.transpose(1, 2))                 # [BHn, C, C]
        mask = torch.ones(C, C, dtype=dtype, device=q.device).tril()
        a = _MulConstFn.apply(a, mask)
        intra = matmul(a, v1c)                               # [BHn, C, d+8]
        # between chunks: exclusive prefix sum of the chunk states (fp32)
        st = matmul(pkc.transpose(1, 2), v1c).reshape(BH, n, d, d + 8).float()
        prefix = torch.cumsum(st, 1) - st
        if sp is not None:
            prefix = prefix + sp.exclusive_prefix(st.sum(1))[:, None]      # states of the tokens on lower ranks
        prefix = prefix.to(dtype).reshape(BH * n, d, d + 8)
        inter = matmul(pqc, prefix)                          # [BHn, C, d+8]
        nd = (intra.float() + inter.float()).reshape(BH, Sp, d + 8)[:, :S]
    nd = nd.float()
    out = _DivFn.apply(nd[..., :d], nd[..., d:d + 1] + eps)  # [BH, S, d]
    return out.to(dtype).reshape(B, H, S, d).permute(0, 2, 1, 3)


def linear_attention_ref(q, k, v, scale=1.0, eps=1e-6, causal=False, kind="elu"):
    """O(S^2) fp32 reference (the role of `naive_reference`, src/linear_attention.rs:684-719)."""
    f = (lambda x: torch.where(x > 0, x + 1, torch.exp(x))) if kind == "elu" else (lambda x: torch.relu(x) ** 2)
    pq = f(q.float() * scale).permute(0, 2, 1, 3); pk = f(k.float() * scale).permute(0, 2, 1, 3); vv = v.float().permute(0, 2, 1, 3)
    a = pq @ pk.transpose(-1, -2)
    if causal:
        S = a.shape[-1]
        a = a * torch.ones(S, S, device=a.device).tril()
    out = (a @ vv) / (a.sum(-1, keepdim=True) + eps)
    return out.permute(0, 2, 1, 3)


def linear_attention_forward(q, k, v, batch, seq, d, scale, eps, causal, kind):
    """Flat-buffer form of the reference API (src/linear_attention.rs:110-136): [batch, seq, d] tensors."""
    name = "elu" if int(kind) == 0 else "relu2"
    t = lambda x: torch.as_tensor(x, dtype=torch.float32).reshape(batch, seq, 1, d)
    return linear_attention(t(q), t(k), t(v), scale, eps, causal, name).reshape(batch, seq, d)


def linear_attention_backward(q, k, v, grad, batch, seq, d, scale, eps, causal, kind):
    name = "elu" if int(kind) == 0 else "relu2"
    t = lambda x: torch.as_tensor(x, dtype=torch.float32).reshape(batch, seq, 1, d).clone().requires_grad_(True)
    qq, kk, vv = t(q), t(k), t(v)
    out = linear_attention(qq, kk, vv, scale, eps, causal, name)
    out.backward(torch.as_tensor(grad, dtype=torch.float32).reshape(batch, seq, 1, d))
    return qq.grad.reshape(batch, seq, d), kk.grad.reshape(batch, seq, d), vv.grad.reshape(batch, seq, d)


class LinearAttention:
    """Config struct of the reference (`LinearAttention::new(kind, d).causal(b).with_scale(s)`, src/linear_attention.rs:640-677)."""

    def __init__(self, kind="elu", d: int = 64):
        kind = getattr(kind, "name", kind)
        self.kind = "elu" if (kind in ("elu", "Elu", 0)) else "relu2"
        self.d, self.is_causal, self.scale, self.eps = d, False, 1.0 / math.sqrt(d), 1e-6

    @staticmethod
    def new(kind, d: int) -> "LinearAttention":
        return LinearAttention(kind, d)

    @staticmethod
    def elu(d: int) -> "LinearAttention":
        return LinearAttention("elu", d)

    def causal(self, flag: bool = True):
        self.is_causal = flag; return self

    def with_scale(self, s: float):
        self.scale = s; return self

    def forward(self, q, k, v):
        """[B, S, d] tensors."""
        o = linear_attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), self.scale, self.eps, self.is_causal, self.kind)
        return o.squeeze(2)


LinearAttentionLayer = LinearAttention
