"""CPU stand-in for the reference's own build (csrc/cpu_ref/): its packed AVX2 4x16 `sgemm` with MC/KC/NC = 128/256/256
(rust-nn src/blas.rs:104-186, 429-508), its scalar flash-attention / linear-attention / selective-scan / LayerNorm loops
(src/tensor.rs:633-662, 859-878, 1027-1046; src/linear_attention.rs:139-266), its AVX2 Adam (src/optim.rs:121-168) and a
whole MLP training step on top of them. The reference is a Rust crate and needs a toolchain this package does not
assume; these C++ restatements serve as independent fp32 oracles for the CUDA kernels and as the timed CPU baseline for
the shapes the reference publishes numbers on (`bench_configs.py ref_mlp`)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _native as nv

_F, _I = C.POINTER(C.c_float), C.POINTER(C.c_int)
nv.register_sigs({
    "b200_cpu_sgemm": [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_int],
    "b200_cpu_flash_attention": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int],
    "b200_cpu_linear_attention": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int],
    "b200_cpu_selective_scan": [C.c_void_p] * 6 + [C.c_int] * 4,
    "b200_cpu_layernorm": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_float],
    "b200_cpu_adam": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_float, C.c_float, C.c_float, C.c_float],
    "b200_cpu_fused_linear": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int],
    "b200_cpu_mlp_step": [C.c_int, C.c_void_p] + [C.c_void_p] * 6 + [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_void_p],
})


def _f32(t):
    return t.detach().to(torch.float32).contiguous().cpu()


def sgemm(a: torch.Tensor, b: torch.Tensor, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None, threads: int = 0) -> torch.Tensor:
    """alpha * op(a) @ op(b) + beta * c on the packed AVX2 kernel (row-major fp32)."""
    a, b = _f32(a), _f32(b)
    m, k = (a.shape[1], a.shape[0]) if trans_a else a.shape
    kb, n = (b.shape[1], b.shape[0]) if trans_b else b.shape
    if k != kb:
        raise ValueError("inner dimensions differ")
    out = torch.zeros(m, n) if c is None else _f32(c).clone()
    nv.check(nv.host().b200_cpu_sgemm(int(trans_a), int(trans_b), m, n, k, alpha, a.data_ptr(), a.shape[1], b.data_ptr(), b.shape[1],
                                      beta, out.data_ptr(), n, threads), "cpu_sgemm")
    return out


def flash_attention(q, k, v, scale=None, causal=False):
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, S, d = q.shape
    out = torch.empty_like(q)
    nv.check(nv.host().b200_cpu_flash_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, d,
                                                float(scale if scale is not None else d ** -0.5), int(causal)), "cpu_flash")
    return out


def linear_attention(q, k, v, scale=1.0, eps=1e-6, causal=False, kind="elu"):
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, S, d = q.shape
    out = torch.empty_like(q)
    nv.check(nv.host().b200_cpu_linear_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, d, float(scale), float(eps),
                                                 int(causal), 0 if kind == "elu" else 1), "cpu_linear_attention")
    return out


def selective_scan(u, delta, A, Bm, Cm):
    u, delta, A, Bm, Cm = (_f32(t) for t in (u, delta, A, Bm, Cm))
    B, S, D = u.shape
    y = torch.empty_like(u)
    nv.check(nv.host().b200_cpu_selective_scan(u.data_ptr(), delta.data_ptr(), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(), y.data_ptr(),
                                               B, S, D, A.shape[1]), "cpu_scan")
    return y


def layer_norm(x, gamma, beta, eps=1e-5):
    x, gamma, beta = _f32(x), _f32(gamma), _f32(beta)
    y = torch.empty_like(x)
    nv.check(nv.host().b200_cpu_layernorm(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), x.numel() // x.shape[-1], x.shape[-1], eps), "cpu_ln")
    return y


def adam_update(p, g, m, v, b1, b2, eps, lr_t):
    """In place on contiguous fp32 CPU tensors (the contract of `adam_update_avx2`, src/optim.rs:121-168)."""
    nv.check(nv.host().b200_cpu_adam(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), b1, b2, eps, lr_t), "cpu_adam")


def fused_linear(x, w, b=None, act="none"):
    x, w = _f32(x), _f32(w)
    bb = _f32(b) if b is not None else None
    y = torch.empty(x.shape[0], w.shape[0])
    nv.check(nv.host().b200_cpu_fused_linear(x.data_ptr(), w.data_ptr(), bb.data_ptr() if bb is not None else None, y.data_ptr(),
                                             x.shape[0], x.shape[1], w.shape[0], 1 if act == "relu" else 0), "cpu_fused_linear")
    return y


class CpuMLP:
    """ReLU MLP trained by `b200_cpu_mlp_step`: forward, loss, backward and Adam in one native call per step."""

    def __init__(self, dims, seed: int = 0, init: str = "he"):
        g = torch.Generator().manual_seed(seed)
        self.dims = list(dims)
        L = len(dims) - 1
        if init == "he":
            self.W = [(torch.randn(dims[i + 1], dims[i], generator=g) * (2.0 / dims[i]) ** 0.5).contiguous() for i in range(L)]
        else:                                                  # Kaiming-uniform (the MLP benchmark configuration)
            self.W = [((torch.rand(dims[i + 1], dims[i], generator=g) * 2 - 1) / dims[i] ** 0.5).contiguous() for i in range(L)]
        self.b = [torch.zeros(dims[i + 1]) for i in range(L)]
        z = lambda ts: [torch.zeros_like(t) for t in ts]
        self.mW, self.vW, self.mb, self.vb = z(self.W), z(self.W), z(self.b), z(self.b)
        self.steps = 0
        arr = lambda ts: (C.c_void_p * L)(*[t.data_ptr() for t in ts])
        self._ptrs = [arr(t) for t in (self.W, self.b, self.mW, self.vW, self.mb, self.vb)]
        self._dims = (C.c_int * (L + 1))(*self.dims)

    def step(self, x: torch.Tensor, labels=None, targets=None, lr: float = 1e-3, threads: int = 1) -> float:
        x = _f32(x)
        L = len(self.dims) - 1
        loss = C.c_float(0)
        lab = labels.to(torch.int32).contiguous() if labels is not None else None
        tg = _f32(targets) if targets is not None else None
        nv.check(nv.host().b200_cpu_mlp_step(L, self._dims, *self._ptrs, x.data_ptr(), lab.data_ptr() if lab is not None else None,
                                             tg.data_ptr() if tg is not None else None, x.shape[0], 0 if labels is not None else 1,
                                             lr, self.steps, threads, C.byref(loss)), "cpu_mlp_step")
        self.steps += 1
        return float(loss.value)
