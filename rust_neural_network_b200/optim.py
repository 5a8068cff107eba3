"""Optimizers (rust-nn src/optim.rs:5-314): SGD, Adam, RMSprop, Muon behind the reference's
`Optimizer` interface (`step`, `zero_grad`).

All parameters of one optimizer are re-homed into ONE flat fp32 buffer (`FlatParams`): master
weights, gradients and optimizer state are contiguous, every parameter's `.data` / `.grad` becomes a
view, and a step is a single kernel launch that also writes the bf16 shadow weights. The flat
gradient buffer is what the data-parallel reduce-scatter operates on. Step counters live on the
device so a step can be captured in a CUDA graph.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .ops import kernels as K
from .ops.gemm import gemm

_ALIGN = 64   # elements; keeps every parameter 256-byte aligned inside the flat buffers


from ._compat import NewMixin as _NewMixin  # noqa: E402

class FlatParams:
    """Flat fp32 master / grad buffers and a flat bf16 shadow for a list of parameters.

    Parameters tagged with the same ``_fuse_group`` object are laid out back to back in the order
    of their ``_fuse_index`` (no padding between them) so that, e.g., the Q, K and V projection
    weights form one contiguous [3d, d] matrix for a fused GEMM."""

    def __init__(self, params: Sequence[torch.nn.Parameter], with_shadow: bool = True, pad_to: int = 1):
        params = [p for p in params]
        assert params, "no parameters"
        dev = params[0].device
        order: List[torch.nn.Parameter] = []
        placed = set()
        groups = {}
        for p in params:
            g = getattr(p, "_fuse_group", None)
            if g is not None:
                groups.setdefault(id(g), []).append(p)
        for p in params:
            if id(p) in placed:
                continue
            g = getattr(p, "_fuse_group", None)
            if g is None:
                order.append(p); placed.add(id(p))
            else:
                for q in sorted(groups[id(g)], key=lambda t: t._fuse_index):
                    if id(q) not in placed:
                        order.append(q); placed.add(id(q))
        offsets, off = {}, 0
        prev_group = None
        for p in order:
            g = getattr(p, "_fuse_group", None)
            if g is None or g is not prev_group:
                off = (off + _ALIGN - 1) // _ALIGN * _ALIGN
            offsets[id(p)] = off
            off += p.numel()
            prev_group = g
        total = (off + _ALIGN - 1) // _ALIGN * _ALIGN
        if pad_to > 1:
            total = (total + pad_to - 1) // pad_to * pad_to
        self.params = params
        self.order = order
        self.offsets = offsets
        self.numel = total
        self.device = dev
        self.master = torch.zeros(total, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(total, dtype=torch.float32, device=dev)
        self.shadow = torch.zeros(total, dtype=torch.bfloat16, device=dev) if with_shadow else None
        with torch.no_grad():
            for p in order:
                o, n = offsets[id(p)], p.numel()
                self.master[o:o + n].copy_(p.data.reshape(-1))
                old_grad = p.grad
                p.data = self.master[o:o + n].view(p.shape)
                p.grad = self.grad[o:o + n].view(p.shape)
                if old_grad is not None:
                    p.grad.copy_(old_grad)
                p._fused_grad = True
                if with_shadow:
                    p._lp = self.shadow[o:o + n].view(p.shape)
                    p._lp_version = p._version
            if with_shadow:
                self.shadow.copy_(self.master)

    def segments(self) -> torch.Tensor:
        """int64 [nseg, 2] table of [begin, end) element ranges of the parameters in layout order
        (alignment padding between parameters belongs to no segment)."""
        offs = [[self.offsets[id(p)], self.offsets[id(p)] + p.numel()] for p in self.order]
        return torch.tensor(offs, dtype=torch.int64, device=self.device)

    def refresh_views(self):
        """Re-establish `.grad` views (something set them to None) and shadow versions."""
        for p in self.order:
            o, n = self.offsets[id(p)], p.numel()
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * o:
                p.grad = self.grad[o:o + n].view(p.shape)
            p._lp_version = p._version


class Optimizer(_NewMixin):
    """`step()` consumes the gradients, `zero_grad()` clears them (src/optim.rs:5-9)."""

    def __init__(self, params, lr: float):
        self.params = [p for p in params if p.requires_grad]
        self.lr = float(lr)
        self.flat = FlatParams(self.params)
        dev = self.flat.device
        self.step_t = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_scale: Optional[torch.Tensor] = None     # optional 1-element device multiplier (clipping)
        self._scalars = torch.zeros(4, dtype=torch.float32, device=dev)

    def zero_grad(self):
        self.flat.refresh_views()
        self.flat.grad.zero_()

    def clip_grad_norm(self, max_norm: float) -> torch.Tensor:
        """Global-norm clipping folded into the next `step()` (no host sync): computes the norm of the
        flat gradient on the device and stores the coefficient the update kernel multiplies by.
        Returns the 0-d device tensor holding the norm (rust-nn src/distributed.rs:507-523)."""
        self._scalars.zero_()
        K.reduce_all(self.flat.grad, "sumsq", out=self._scalars[0:1])
        K.clip_coef(self._scalars, max_norm)
        self.grad_scale = self._scalars[1:2]
        return self._scalars[2]

    def set_lr(self, lr: float):
        self.lr = float(lr)

    def state_tensors(self) -> dict:
        return {"step": self.step_t}

    def snapshot_tensors(self) -> list:
        """Every tensor a step changes (weights, shadows, optimizer state): what `Trainer.capture` saves before its
        warm-up steps and restores after them."""
        flat = getattr(self, "flat", None)
        ts = []
        if flat is not None:
            ts.append(flat.master)
            if flat.shadow is not None:
                ts.append(flat.shadow)
        return ts + [t for t in self.state_tensors().values() if isinstance(t, torch.Tensor)]

    def step(self):
        raise NotImplementedError


class MultiOptimizer(Optimizer):
    """Several optimizers stepped as one (e.g. a tensor-parallel model: a sharded data-parallel optimizer for the
    replicated parameters next to a local one for the parameters each rank owns outright)."""

    def __init__(self, optimizers: Sequence[Optimizer]):
        self.opts = list(optimizers)
        self.params = [p for o in self.opts for p in o.params]
        self.flat = None
        self.lr = self.opts[0].lr

    def zero_grad(self):
        for o in self.opts:
            o.zero_grad()

    def step(self):
        for o in self.opts:
            o.step()

    def set_lr(self, lr: float):
        self.lr = float(lr)
        for o in self.opts:
            o.set_lr(lr)

    def clip_grad_norm(self, max_norm: float):
        raise NotImplementedError("a global norm across several optimizers is not implemented")

    def state_tensors(self) -> dict:
        return {f"{k}@{j}": v for j, o in enumerate(self.opts) for k, v in o.state_tensors().items()}

    def snapshot_tensors(self) -> list:
        return [t for o in self.opts for t in o.snapshot_tensors()]

    def prepare_checkpoint(self):
        for o in self.opts:
            if hasattr(o, "prepare_checkpoint"):
                o.prepare_checkpoint()


class SGD(Optimizer):
    """buf = g on the first step, then momentum*buf + g; p -= lr*buf (src/optim.rs:29-47)."""

    def __init__(self, params, lr: float, momentum: float = 0.0):
        super().__init__(params, lr)
        self.momentum = float(momentum)
        self.buf = torch.zeros_like(self.flat.master) if momentum > 0 else None

    def step(self):
        K.sgd_step(self.flat.master, self.flat.grad, self.buf, self.flat.shadow, self.lr, self.momentum, self.step_t, self.grad_scale)

    def state_tensors(self):
        d = {"step": self.step_t}
        if self.buf is not None:
            d["momentum"] = self.buf
        return d


class Adam(Optimizer):
    """Adam with b=(0.9, 0.999), eps 1e-8. The default form is the reference's
    (`lr_t = lr*sqrt(1-b2^t)/(1-b1^t)`, `p -= lr_t*m/(sqrt(v)+eps)`, src/optim.rs:170-212);
    `torch_compat=True` switches to PyTorch's `m_hat/(sqrt(v_hat)+eps)`."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 torch_compat: bool = False):
        super().__init__(params, lr)
        self.b1, self.b2 = betas
        self.eps, self.weight_decay, self.torch_compat = eps, weight_decay, torch_compat
        self.m = torch.zeros_like(self.flat.master)
        self.v = torch.zeros_like(self.flat.master)

    def step(self):
        K.adam_step(self.flat.master, self.flat.grad, self.m, self.v, self.flat.shadow, self.lr, self.b1, self.b2,
                    self.eps, self.weight_decay, self.torch_compat, self.step_t, self.grad_scale)

    def state_tensors(self):
        return {"step": self.step_t, "m": self.m, "v": self.v}


class RMSprop(Optimizer):
    """v = a v + (1-a) g^2; p -= lr*g/(sqrt(v)+eps), a=0.99, eps 1e-8 (src/optim.rs:246-256)."""

    def __init__(self, params, lr: float, alpha: float = 0.99, eps: float = 1e-8):
        super().__init__(params, lr)
        self.alpha, self.eps = alpha, eps
        self.v = torch.zeros_like(self.flat.master)

    def step(self):
        K.rmsprop_step(self.flat.master, self.flat.grad, self.v, self.flat.shadow, self.lr, self.alpha, self.eps, self.grad_scale)
        self.step_t.add_(1.0)

    def state_tensors(self):
        return {"step": self.step_t, "v": self.v}


def newton_schulz(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Orthogonalise a 2-D matrix with the quintic Newton-Schulz iteration, all products on the
    tcgen05 GEMM (bf16 operands, fp32 accumulate). Returns fp32 of G's shape."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.float()
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t().contiguous()
    X = X / (X.norm() + 1e-7)
    Xb = X.to(torch.bfloat16) if X.is_cuda else X
    for _ in range(steps):
        A = gemm(Xb, Xb)                                   # X X^T            [m, m]
        B = gemm(A, A, out_dtype=torch.float32 if not Xb.is_cuda else None)   # A A^T = A^2 (A symmetric)
        Bm = (b * A.float() + c * B.float())
        Bm = Bm.to(Xb.dtype)
        Xn = a * Xb.float() + gemm(Bm, Xb, b_mn=True, out_dtype=torch.float32).float()
        Xb = Xn.to(Xb.dtype)
    X = Xb.float()
    return X.t().contiguous() if transposed else X


class Muon(Optimizer):
    """Muon. `mode="rms"` (default) is the reference's variant: the gradient of each tensor is
    divided by its RMS, then momentum SGD (src/optim.rs:284-307; it has no Newton-Schulz step).
    `mode="newton_schulz"` orthogonalises the momentum of every 2-D parameter with a quintic
    Newton-Schulz iteration on the tcgen05 GEMM (other parameters use the RMS rule)."""

    def __init__(self, params, lr: float, momentum: float = 0.95, mode: str = "rms", ns_steps: int = 5):
        super().__init__(params, lr)
        self.momentum, self.mode, self.ns_steps = float(momentum), mode, ns_steps
        self.buf = torch.zeros_like(self.flat.master)
        self.seg = self.flat.segments()
        self._scratch = torch.zeros(self.seg.shape[0], dtype=torch.float32, device=self.flat.device)

    def step(self):
        if self.mode == "rms":
            K.muon_rms_step(self.flat.master, self.flat.grad, self.buf, self.flat.shadow, self.seg, self.lr,
                            self.momentum, 1e-8, self._scratch)
            self.step_t.add_(1.0)
            return
        with torch.no_grad():
            self.buf.mul_(self.momentum).add_(self.flat.grad)
            for p in self.flat.order:
                o, n = self.flat.offsets[id(p)], p.numel()
                m = self.buf[o:o + n].view(p.shape)
                if p.dim() == 2 and min(p.shape) > 1:
                    upd = newton_schulz(m, self.ns_steps) * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                else:
                    upd = m / (m.pow(2).mean().sqrt().clamp_min(1e-8))
                p.data.add_(upd, alpha=-self.lr)
            if self.flat.shadow is not None:
                self.flat.shadow.copy_(self.flat.master)
            self.step_t.add_(1.0)

    def state_tensors(self):
        return {"step": self.step_t, "momentum": self.buf}


def adam_update_scalar(g, m, v, d, b1, b2, one_minus_b1, one_minus_b2, eps, lr_t):
    """The reference's scalar Adam kernel contract on flat tensors, in place
    (rust-nn src/optim.rs:91-111): m,v updated; d -= lr_t * m / (sqrt(v) + eps)."""
    m.mul_(b1).add_(g, alpha=one_minus_b1)
    v.mul_(b2).addcmul_(g, g, value=one_minus_b2)
    d.addcdiv_(m, v.sqrt().add_(eps), value=-lr_t)


adam_update_avx2 = adam_update_scalar   # same contract; the vector path here is the CUDA kernel
