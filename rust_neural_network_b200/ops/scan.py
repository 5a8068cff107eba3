"""Mamba ops: selective scan (S6) and depthwise causal conv1d, forward and backward on the
sm_100a kernels of csrc/scan/scan.cu, with fp32 PyTorch references (used on CPU and as test oracles).

Shapes follow rust-nn `Tensor::selective_scan(delta, b_vec, c_vec, u, a)` (src/tensor.rs:833):
u, delta [B, S, D]; B_t, C_t [B, S, N]; A [D, N] -> y [B, S, D]; and
`Tensor::conv1d_causal(input [B, S, C], weight [C, K])` (src/tensor.rs:903). Extensions used by the
Mamba configuration: a D skip term, a delta bias with softplus inside the kernel, a fused SiLU gate z,
a conv bias and a fused SiLU after the convolution.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch.autograd import Function

from .. import _native as nv

SCAN_CK = 8   # checkpoint interval of the kernels (csrc/scan/scan.cu: SCAN_CK)
SCAN_MAX_N = 16


class ScanArgs(C.Structure):
    _fields_ = [
        ("u", C.c_void_p), ("u_ld", C.c_longlong), ("delta", C.c_void_p), ("delta_ld", C.c_longlong),
        ("z", C.c_void_p), ("z_ld", C.c_longlong), ("Bm", C.c_void_p), ("b_ld", C.c_longlong),
        ("Cm", C.c_void_p), ("c_ld", C.c_longlong), ("A", C.c_void_p), ("Dskip", C.c_void_p), ("delta_bias", C.c_void_p),
        ("y", C.c_void_p), ("y_ld", C.c_longlong), ("hck", C.c_void_p),
        ("B", C.c_int), ("S", C.c_int), ("D", C.c_int), ("N", C.c_int), ("delta_softplus", C.c_int),
        ("dy", C.c_void_p), ("dy_ld", C.c_longlong), ("du", C.c_void_p), ("du_ld", C.c_longlong),
        ("ddelta", C.c_void_p), ("ddelta_ld", C.c_longlong), ("dz", C.c_void_p), ("dz_ld", C.c_longlong),
        ("dB", C.c_void_p), ("dC", C.c_void_p), ("dA", C.c_void_p), ("dDskip", C.c_void_p), ("ddelta_bias", C.c_void_p),
    ]


nv.register_sigs({
    "b200_selective_scan_fwd": [C.POINTER(ScanArgs), C.c_int, C.c_void_p],
    "b200_selective_scan_bwd": [C.POINTER(ScanArgs), C.c_int, C.c_void_p],
    "b200_conv1d_fwd": [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
    "b200_conv1d_bwd": [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p,
                        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
})


# ----------------------------------------------------------------------------- references
def selective_scan_ref(u, delta, A, Bm, Cm, Dskip=None, z=None, delta_bias=None, delta_softplus=False):
    """Sequential fp32 reference of the recurrence."""
    uf, df = u.float(), delta.float()
    if delta_bias is not None:
        df = df + delta_bias.float()
    if delta_softplus:
        df = torch.nn.functional.softplus(df, threshold=20.0)
    Bf, Cf, Af = Bm.float(), Cm.float(), A.float()
    Bsz, S, D = uf.shape
    h = torch.zeros(Bsz, D, Af.shape[1], dtype=torch.float32, device=u.device)
    ys = []
    for t in range(S):
        da = torch.exp(df[:, t, :, None] * Af[None])
        h = da * h + (df[:, t] * uf[:, t])[:, :, None] * Bf[:, t, None, :]
        ys.append((h * Cf[:, t, None, :]).sum(-1))
    y = torch.stack(ys, 1)
    if Dskip is not None:
        y = y + uf * Dskip.float()
    if z is not None:
        y = y * torch.nn.functional.silu(z.float())
    return y.to(u.dtype)


def causal_conv1d_ref(x, w, bias=None, act="none"):
    """x [B, S, C], w [C, K]: y[b,t,c] = sum_k w[c,k] x[b, t-(K-1)+k, c] (+ bias) (then SiLU)."""
    Kw = w.shape[1]
    xp = torch.nn.functional.pad(x.float().transpose(1, 2), (Kw - 1, 0))
    y = torch.nn.functional.conv1d(xp, w.float()[:, None, :], bias.float() if bias is not None else None, groups=w.shape[0]).transpose(1, 2)
    if act == "silu":
        y = torch.nn.functional.silu(y)
    return y.to(x.dtype)


# ----------------------------------------------------------------------------- raw launchers
def _rows(t):
    """[B, S, X] tensor with unit inner stride and batch stride = S * row stride -> (tensor, ld)."""
    if t.stride(2) != 1 or t.stride(0) != t.shape[1] * t.stride(1):
        t = t.contiguous()
    return t, t.stride(1)


def _isbf(t):
    if t.dtype == torch.bfloat16: return 1
    if t.dtype == torch.float32: return 0
    raise TypeError("scan kernels take bf16 or fp32")


@nv.traced("selective_scan")
def scan_fwd_raw(u, delta, A, Bm, Cm, Dskip, z, delta_bias, delta_softplus, save_ck):
    Bsz, S, D = u.shape
    N = A.shape[1]
    if N > SCAN_MAX_N:
        raise ValueError(f"d_state {N} > {SCAN_MAX_N}")
    u, u_ld = _rows(u); delta, d_ld = _rows(delta.to(u.dtype)); Bm, b_ld = _rows(Bm.to(u.dtype)); Cm, c_ld = _rows(Cm.to(u.dtype))
    z_ld = 0
    if z is not None:
        z, z_ld = _rows(z.to(u.dtype))
    y = torch.empty((Bsz, S, D), dtype=u.dtype, device=u.device)
    n_ck = (S + SCAN_CK - 1) // SCAN_CK
    hck = torch.empty((Bsz, n_ck, D, N), dtype=torch.float32, device=u.device) if save_ck else None
    a = ScanArgs()
    a.u, a.u_ld, a.delta, a.delta_ld = u.data_ptr(), u_ld, delta.data_ptr(), d_ld
    a.z, a.z_ld = nv.ptr(z), z_ld
    a.Bm, a.b_ld, a.Cm, a.c_ld = Bm.data_ptr(), b_ld, Cm.data_ptr(), c_ld
    Af = A if (A.dtype == torch.float32 and A.is_contiguous()) else A.float().contiguous()
    a.A = Af.data_ptr()
    a.Dskip, a.delta_bias = nv.ptr(Dskip), nv.ptr(delta_bias)
    a.y, a.y_ld, a.hck = y.data_ptr(), D, nv.ptr(hck)
    a.B, a.S, a.D, a.N, a.delta_softplus = Bsz, S, D, N, int(delta_softplus)
    nv.check(nv.cuda().b200_selective_scan_fwd(C.byref(a), _isbf(u), nv.stream_ptr()), "selective_scan_fwd")
    nv.count_launch()
    return y, hck


@nv.traced("selective_scan")
def scan_bwd_raw(dy, u, delta, A, Bm, Cm, Dskip, z, delta_bias, delta_softplus, hck):
    Bsz, S, D = u.shape
    N = A.shape[1]
    dev = u.device
    u, u_ld = _rows(u); delta, d_ld = _rows(delta.to(u.dtype)); Bm, b_ld = _rows(Bm.to(u.dtype)); Cm, c_ld = _rows(Cm.to(u.dtype))
    dy, dy_ld = _rows(dy.to(u.dtype))
    z_ld = 0
    if z is not None:
        z, z_ld = _rows(z.to(u.dtype))
    du = torch.empty((Bsz, S, D), dtype=u.dtype, device=dev)
    ddelta = torch.empty((Bsz, S, D), dtype=u.dtype, device=dev)
    dz = torch.empty((Bsz, S, D), dtype=u.dtype, device=dev) if z is not None else None
    dB = torch.zeros((Bsz, S, N), dtype=torch.float32, device=dev)
    dC = torch.zeros((Bsz, S, N), dtype=torch.float32, device=dev)
    dA = torch.zeros((D, N), dtype=torch.float32, device=dev)
    dD = torch.zeros(D, dtype=torch.float32, device=dev) if Dskip is not None else None
    ddb = torch.zeros(D, dtype=torch.float32, device=dev) if delta_bias is not None else None
    Af = A if (A.dtype == torch.float32 and A.is_contiguous()) else A.float().contiguous()
    a = ScanArgs()
    a.u, a.u_ld, a.delta, a.delta_ld = u.data_ptr(), u_ld, delta.data_ptr(), d_ld
    a.z, a.z_ld = nv.ptr(z), z_ld
    a.Bm, a.b_ld, a.Cm, a.c_ld = Bm.data_ptr(), b_ld, Cm.data_ptr(), c_ld
    a.A, a.Dskip, a.delta_bias = Af.data_ptr(), nv.ptr(Dskip), nv.ptr(delta_bias)
    a.y, a.y_ld, a.hck = 0, D, hck.data_ptr()
    a.B, a.S, a.D, a.N, a.delta_softplus = Bsz, S, D, N, int(delta_softplus)
    a.dy, a.dy_ld, a.du, a.du_ld = dy.data_ptr(), dy_ld, du.data_ptr(), D
    a.ddelta, a.ddelta_ld, a.dz, a.dz_ld = ddelta.data_ptr(), D, nv.ptr(dz), D
    a.dB, a.dC, a.dA, a.dDskip, a.ddelta_bias = dB.data_ptr(), dC.data_ptr(), dA.data_ptr(), nv.ptr(dD), nv.ptr(ddb)
    nv.check(nv.cuda().b200_selective_scan_bwd(C.byref(a), _isbf(u), nv.stream_ptr()), "selective_scan_bwd")
    nv.count_launch()
    return du, ddelta, dA, dB, dC, dD, dz, ddb


# ----------------------------------------------------------------------------- autograd
class SelectiveScanFn(Function):
    @staticmethod
    def forward(ctx, u, delta, A, Bm, Cm, Dskip, z, delta_bias, delta_softplus, recompute=False):
        ctx.recompute = bool(recompute)
        if not u.is_cuda:
            ctx.cpu = True
            ctx.save_for_backward(u, delta, A, Bm, Cm, Dskip, z, delta_bias)
            ctx.softplus = delta_softplus
            return selective_scan_ref(u, delta, A, Bm, Cm, Dskip, z, delta_bias, delta_softplus)
        ctx.cpu = False
        need = any(t is not None and t.requires_grad for t in (u, delta, A, Bm, Cm, Dskip, z, delta_bias))
        # recompute: the state checkpoints (B x S/8 x D x N fp32, 4x the size of u) are not kept; the backward runs the
        # forward kernel once more to rebuild them, so only one layer's checkpoints exist at a time
        y, hck = scan_fwd_raw(u, delta, A.detach(), Bm, Cm, Dskip.detach() if Dskip is not None else None, z,
                              delta_bias.detach() if delta_bias is not None else None, delta_softplus, need and not ctx.recompute)
        ctx.save_for_backward(u, delta, A, Bm, Cm, Dskip, z, delta_bias, hck)
        ctx.softplus = delta_softplus
        return y

    @staticmethod
    def backward(ctx, dy):
        if ctx.cpu:
            u, delta, A, Bm, Cm, Dskip, z, delta_bias = ctx.saved_tensors
            with torch.enable_grad():
                ins = [t.detach().float().requires_grad_(True) if t is not None else None for t in (u, delta, A, Bm, Cm, Dskip, z, delta_bias)]
                y = selective_scan_ref(*ins, ctx.softplus)
                live = [t for t in ins if t is not None]
                grads = torch.autograd.grad(y, live, dy.float(), allow_unused=True)
            it = iter(grads)
            outs = []
            for t, orig in zip(ins, (u, delta, A, Bm, Cm, Dskip, z, delta_bias)):
                g = next(it) if t is not None else None
                outs.append(g.to(orig.dtype) if g is not None else None)
            return (*outs, None, None)
        u, delta, A, Bm, Cm, Dskip, z, delta_bias, hck = ctx.saved_tensors
        if hck is None:
            _, hck = scan_fwd_raw(u, delta, A.detach(), Bm, Cm, Dskip.detach() if Dskip is not None else None, z,
                                  delta_bias.detach() if delta_bias is not None else None, ctx.softplus, True)
        du, ddelta, dA, dB, dC, dD, dz, ddb = scan_bwd_raw(dy, u, delta, A.detach(), Bm, Cm,
                                                           Dskip.detach() if Dskip is not None else None, z,
                                                           delta_bias.detach() if delta_bias is not None else None,
                                                           ctx.softplus, hck)
        return (du, ddelta.to(delta.dtype), dA.to(A.dtype), dB.to(Bm.dtype), dC.to(Cm.dtype),
                dD.to(Dskip.dtype) if dD is not None else None, dz, ddb.to(delta_bias.dtype) if ddb is not None else None, None, None)


def selective_scan(u, delta, A, Bm, Cm, Dskip=None, z=None, delta_bias=None, delta_softplus=False, recompute=False):
    """`recompute=True` trades one more forward scan in the backward pass for not keeping the state checkpoints of
    every layer alive between forward and backward (4x the bytes of `u` per layer)."""
    if z is not None and u.is_cuda and A.shape[1] == 16:
        # the lane-per-state kernels (16 states) take no gate: y * silu(z) is one elementwise kernel on each side of them,
        # far cheaper than falling back to the thread-per-channel scan that fuses it
        from . import functional as F
        return F.mul_silu(SelectiveScanFn.apply(u, delta, A, Bm, Cm, Dskip, None, delta_bias, delta_softplus, recompute), z.to(u.dtype))
    return SelectiveScanFn.apply(u, delta, A, Bm, Cm, Dskip, z, delta_bias, delta_softplus, recompute)


class CausalConv1dFn(Function):
    @staticmethod
    def forward(ctx, x, w, bias, act):
        ctx.act = act
        ctx.save_for_backward(x, w, bias)
        if not x.is_cuda:
            return causal_conv1d_ref(x, w, bias, act)
        Bsz, S, Cc = x.shape
        xr, x_ld = _rows(x)
        y = torch.empty((Bsz, S, Cc), dtype=x.dtype, device=x.device)
        wf = w.detach().float().contiguous()
        bf = bias.detach().float().contiguous() if bias is not None else None
        nv.check(nv.cuda().b200_conv1d_fwd(xr.data_ptr(), x_ld, wf.data_ptr(), nv.ptr(bf), y.data_ptr(), Cc, Bsz, S, Cc, w.shape[1],
                                           1 if act == "silu" else 0, _isbf(x), nv.stream_ptr()), "conv1d_fwd")
        nv.count_launch()
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, bias = ctx.saved_tensors
        if not x.is_cuda:
            with torch.enable_grad():
                xr = x.detach().float().requires_grad_(True); wr = w.detach().float().requires_grad_(True)
                br = bias.detach().float().requires_grad_(True) if bias is not None else None
                y = causal_conv1d_ref(xr, wr, br, ctx.act)
                gs = torch.autograd.grad(y, [t for t in (xr, wr, br) if t is not None], dy.float())
            return gs[0].to(x.dtype), gs[1].to(w.dtype), (gs[2].to(bias.dtype) if bias is not None else None), None
        Bsz, S, Cc = x.shape
        xr, x_ld = _rows(x); dyr, dy_ld = _rows(dy.to(x.dtype))
        dx = torch.empty((Bsz, S, Cc), dtype=x.dtype, device=x.device)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        db = torch.zeros(Cc, dtype=torch.float32, device=x.device) if bias is not None else None
        wf = w.detach().float().contiguous()
        bf = bias.detach().float().contiguous() if bias is not None else None
        nv.check(nv.cuda().b200_conv1d_bwd(xr.data_ptr(), x_ld, wf.data_ptr(), nv.ptr(bf), dyr.data_ptr(), dy_ld, dx.data_ptr(), Cc,
                                           dw.data_ptr(), nv.ptr(db), Bsz, S, Cc, w.shape[1], 1 if ctx.act == "silu" else 0,
                                           _isbf(x), nv.stream_ptr()), "conv1d_bwd")
        nv.count_launch()
        return dx, dw.to(w.dtype), (db.to(bias.dtype) if db is not None else None), None


def causal_conv1d(x, w, bias=None, act="none"):
    return CausalConv1dFn.apply(x, w, bias, act)
