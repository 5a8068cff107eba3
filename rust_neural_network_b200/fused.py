"""Fused forward ops (rust-nn src/fused.rs): `FusedActivation`, `fused_linear`, `sparse_topk_route`.

`fused_linear` is one GEMM launch whose epilogue adds the bias and applies the activation
(the reference loops over outputs with a SIMD dot product, src/fused.rs:25-138). It is
forward-only like the reference's; the differentiable version is `ops.functional.linear`.
`sparse_topk_route` is the MoE router kernel restricted to its routing outputs: softmax over the
top-k logits of each row (src/fused.rs:145-184), ties resolved towards the lower expert index.
"""
from __future__ import annotations

import enum
from typing import Optional, Tuple

import torch

from .ops import gemm as G


class FusedActivation(enum.Enum):
    None_ = "none"
    ReLU = "relu"
    GELU = "gelu"
    Sigmoid = "sigmoid"


FusedActivation.NONE = FusedActivation.None_


def fused_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 activation: FusedActivation = FusedActivation.None_, out_dtype=None) -> torch.Tensor:
    """act(x W^T + b) for x [batch, in], W [out, in]; result carries no autograd history."""
    act = activation.value if isinstance(activation, FusedActivation) else str(activation).lower()
    x2, w = x.detach(), weight.detach()
    if x2.is_cuda and x2.dtype != w.dtype:
        w = w.to(x2.dtype)
    b = bias.detach() if bias is not None else None
    if b is not None and b.dtype not in (torch.float32, torch.bfloat16):
        b = b.float()
    return G.gemm(x2.reshape(-1, x2.shape[-1]), w, bias=b, act=act, out_dtype=out_dtype or x2.dtype).reshape(*x2.shape[:-1], w.shape[0])


def sparse_topk_route(gating_logits: torch.Tensor, batch: int, num_experts: int, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(indices [batch*k] int64, weights [batch*k] fp32): the k largest logits of each row, in
    descending order, with a softmax over just those k."""
    logits = gating_logits.detach().reshape(batch, num_experts)
    if logits.is_cuda:
        from .models.moe import RouterFn
        idx, w, _counts, _aux = RouterFn.apply(logits.float().contiguous(), k, True, 0.0)
        # softmax over the top-k logits == full softmax renormalised over the chosen k
        return idx.reshape(-1).long(), w.reshape(-1).float()
    vals, idx = torch.topk(logits.float(), k, dim=-1)
    w = torch.softmax(vals, dim=-1)
    return idx.reshape(-1), w.reshape(-1)


from ._compat import install as _install  # noqa: E402

_install(globals())
