"""Linear attention (rust-nn src/linear_attention.rs): feature maps phi = ELU+1 or ReLU^2,
causal and non-causal, forward and backward.

    out_t = phi(s q_t) . S_t / (phi(s q_t) . z_t + eps),   S_t = sum_{u<=t} phi(s k_u) (x) v_u,  z_t = sum_{u<=t} phi(s k_u)

(non-causal: the sums run over the whole sequence). The reference computes the causal form as a
per-token rank-1 recurrence and its backward stores all seq*d^2 states (src/linear_attention.rs:214-266,
502-632). Here the causal form is CHUNKED: tokens are grouped into chunks of C; inside a chunk the
masked C x C product (phi Q)(phi K)^T is applied to [V | 1] (the extra ones column yields the
denominator for free), between chunks a d x (d+8) state is carried by an exclusive prefix sum.

On a GPU the causal bf16 form with head_dim 64 or 128 runs on the FUSED chunk kernels of
csrc/attention/linattn_sm100.cu (`FusedCausalLinearAttnFn`): phi in the prologue, all products on tcgen05 with the
state in TMEM in fp32, the division in the epilogue, one launch forward and two backward. Everything else (non-causal,
other head sizes, fp32, CPU) takes the composition below, in which every
product is a batched call of the tcgen05 GEMM kernel (NT for (phi Q)(phi K)^T, TN for the chunk states,
NN for applying them); the feature maps and the mask are this package's elementwise kernels. The
backward is the autograd composition of the same kernels (each GEMM's backward is two more GEMMs).

Inputs are [B, S, H, d] (any strides); output [B, S, H, d].
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

import ctypes as C

from .. import _native as nv
from . import kernels as K
from .functional import matmul

CHUNK = 128


LA_MAX_WORLD = 8


class LaExchange(C.Structure):
    """Mirror of `LaExchange` in csrc/attention/linattn_sm100.cu: the in-kernel exchange of slice totals between the
    ranks of a sequence-parallel group (role 1: publish, role 2: consume; dir 0: from lower ranks, 1: from higher)."""
    _fields_ = [("state", C.c_void_p * LA_MAX_WORLD), ("flags", C.c_void_p * LA_MAX_WORLD), ("acks", C.c_void_p * LA_MAX_WORLD),
                ("prefix", C.c_void_p), ("words", C.c_void_p), ("wait_cycles", C.c_longlong),
                ("rank", C.c_int), ("world", C.c_int), ("dir", C.c_int), ("role", C.c_int)]


class LinAttnArgs(C.Structure):
    _fields_ = [("q", nv.AttnTensor), ("k", nv.AttnTensor), ("v", nv.AttnTensor), ("o", nv.AttnTensor),
                ("dout", nv.AttnTensor), ("dq", nv.AttnTensor), ("dk", nv.AttnTensor), ("dv", nv.AttnTensor), ("o_lo", nv.AttnTensor),
                ("den", C.c_void_p), ("s_in", C.c_void_p), ("s_out", C.c_void_p), ("ds_in", C.c_void_p), ("ds_out", C.c_void_p),
                ("B", C.c_int), ("H", C.c_int), ("S", C.c_int), ("hd", C.c_int), ("scale", C.c_float), ("eps", C.c_float),
                ("kind", C.c_int), ("state_only", C.c_int), ("status", C.c_void_p), ("sx", LaExchange)]


nv.register_sigs({"b200_linattn": [C.POINTER(LinAttnArgs), C.c_int, C.c_void_p], "b200_linattn_init": []})


def _attn_t(t):
    """[B, S, H, d] tensor with unit inner stride -> AttnTensor (strides in elements); TMA wants 16-byte multiples."""
    a = nv.AttnTensor()
    a.ptr, a.sb, a.ss, a.sh = t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)
    return a


def _tma_ok(t):
    return t.stride(3) == 1 and all(t.stride(i) % 8 == 0 for i in range(3)) and t.data_ptr() % 16 == 0


def fused_supported(q, causal) -> bool:
    return bool(causal and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128))


@nv.traced("linear_attention")
def _launch(which, q, k, v, scale, eps, kind, o=None, den=None, dout=None, dq=None, dk=None, dv=None, s_in=None, s_out=None,
            ds_in=None, ds_out=None, state_only=False, o_lo=None, sx=None):
    """`sx = (SPContext, dir, role)` lets the kernel itself exchange the slice totals with the other ranks (see
    `LaExchange`); it returns the local buffer the consume pass leaves the summed state in."""
    B, S, H, d = q.shape
    a = LinAttnArgs()
    prefix = None
    if sx is not None:
        prefix = sx[0].fill_exchange(a.sx, B * H, d * d + d, sx[1], sx[2])
    a.q, a.k, a.v = _attn_t(q), _attn_t(k), _attn_t(v)
    for name, t in (("o", o), ("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv), ("o_lo", o_lo)):
        if t is not None:
            setattr(a, name, _attn_t(t))
    a.den, a.s_in, a.s_out, a.ds_in, a.ds_out = nv.ptr(den), nv.ptr(s_in), nv.ptr(s_out), nv.ptr(ds_in), nv.ptr(ds_out)
    a.B, a.H, a.S, a.hd, a.scale, a.eps = B, H, S, d, float(scale), float(eps)
    a.kind, a.state_only = (0 if kind == "elu" else 1), int(state_only)
    a.status = nv.status_word(q.device).data_ptr()
    nv.check(nv.cuda().b200_linattn(C.byref(a), which, nv.stream_ptr()), "linattn")
    nv.count_launch()
    return prefix


class FusedCausalLinearAttnFn(Function):
    """Causal linear attention on the fused chunk kernels (csrc/attention/linattn_sm100.cu): one forward kernel, two
    backward kernels (dQ in sequence order, dK / dV in reverse order), state carried in fp32, nothing stored per chunk.
    With `sp` the rank's tokens are one slice of a longer sequence: a state-only pass produces the slice's total state,
    one exchange kernel turns the totals into prefixes (suffixes in the backward), and the main pass starts from them."""

    @staticmethod
    def forward(ctx, q, k, v, scale, eps, kind, sp):
        B, S, H, d = q.shape
        q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
        dev = q.device
        o = torch.empty((B, S, H, d), dtype=torch.bfloat16, device=dev)
        den = torch.empty((B, H, S), dtype=torch.float32, device=dev)
        s_in = None
        in_kernel = sp is not None and sp.world > 1 and sp.backend == "fused"
        if sp is not None and sp.world > 1 and not in_kernel:
            tot = torch.empty((B * H, d * d + d), dtype=torch.float32, device=dev)
            _launch(0, q, k, v, scale, eps, kind, s_out=tot, state_only=True)
            s_in = sp._exchange(tot, 0)                         # sum of the lower ranks' totals
        # the backward needs more of O than its bf16 value (see csrc/attention/linattn_sm100.cu: o_lo): keep the remainder
        need_grad = any(t.requires_grad for t in (q, k, v))
        o_lo = torch.empty_like(o) if need_grad else None
        if in_kernel:
            # the state pass publishes this slice's total in peer-mapped memory, the main pass pulls the lower ranks' totals
            # itself: two launches, no exchange kernel, and a (batch, head) starts as soon as ITS states have arrived
            _launch(0, q, k, v, scale, eps, kind, state_only=True, sx=(sp, 0, 1))
            pre = _launch(0, q, k, v, scale, eps, kind, o=o, den=den, o_lo=o_lo, sx=(sp, 0, 2))
            s_in = pre.clone() if (sp.rank > 0 and need_grad) else None      # the buffer is reused by the next call
        else:
            _launch(0, q, k, v, scale, eps, kind, o=o, den=den, s_in=s_in, o_lo=o_lo)
        ctx.save_for_backward(q, k, v, o, den, s_in if s_in is not None else torch.empty(0), o_lo if o_lo is not None else torch.empty(0))
        ctx.cfg = (scale, eps, kind, sp)
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, den, s_in, o_lo = ctx.saved_tensors
        scale, eps, kind, sp = ctx.cfg
        s_in = s_in if s_in.numel() else None
        o_lo = o_lo if o_lo.numel() else None
        B, S, H, d = q.shape
        dout = dout if (_tma_ok(dout) and dout.dtype == torch.bfloat16) else dout.to(torch.bfloat16).contiguous()
        dq, dk, dv = torch.empty_like(o), torch.empty_like(o), torch.empty_like(o)
        _launch(1, q, k, v, scale, eps, kind, o=o, den=den, dout=dout, dq=dq, s_in=s_in, o_lo=o_lo)
        ds_in = None
        if sp is not None and sp.world > 1 and sp.backend == "fused":
            _launch(2, q, k, v, scale, eps, kind, o=o, den=den, dout=dout, state_only=True, o_lo=o_lo, sx=(sp, 1, 1))
            _launch(2, q, k, v, scale, eps, kind, o=o, den=den, dout=dout, dk=dk, dv=dv, o_lo=o_lo, sx=(sp, 1, 2))
            return dq, dk, dv, None, None, None, None
        if sp is not None and sp.world > 1:
            tot = torch.empty((B * H, d * d + d), dtype=torch.float32, device=q.device)
            _launch(2, q, k, v, scale, eps, kind, o=o, den=den, dout=dout, ds_out=tot, state_only=True, o_lo=o_lo)
            ds_in = sp._exchange(tot, 1)                        # sum of the higher ranks' totals
        _launch(2, q, k, v, scale, eps, kind, o=o, den=den, dout=dout, dk=dk, dv=dv, ds_in=ds_in, o_lo=o_lo)
        return dq, dk, dv, None, None, None, None


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
    if fused_supported(q, causal) and k.dtype == v.dtype == torch.bfloat16:
        return FusedCausalLinearAttnFn.apply(q, k, v, float(scale), float(eps), kind, sp)
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


def linear_attention_ref(q, k, v, scale=1.0, eps=1e-6, causal=False, kind="elu", feature_dtype=None):
    """O(S^2) fp32 reference (the role of `naive_reference`, src/linear_attention.rs:684-719). `feature_dtype=torch.bfloat16`
    rounds phi(sQ) and phi(sK) to bf16 (straight-through for the gradient) and computes everything else in fp32: the
    function a kernel with bf16 tensor-core operands evaluates. ELU + 1 features sit near 1, where bf16 resolves 2^-8, while
    dQ / dK are differences of nearly equal sums over them, so this rounding alone moves dQ by a few per cent."""
    f = (lambda x: torch.where(x > 0, x + 1, torch.exp(x))) if kind == "elu" else (lambda x: torch.relu(x) ** 2)

    def feat(x):
        p = f(x.float() * scale)
        if feature_dtype is not None:
            p = p + (p.to(feature_dtype).float() - p).detach()
        return p.permute(0, 2, 1, 3)

    pq, pk, vv = feat(q), feat(k), v.float().permute(0, 2, 1, 3)
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


from .._compat import alias_fields as _alias_fields  # noqa: E402

_alias_fields(LinearAttention, kernel="kind")                              # src/linear_attention.rs:640-646
