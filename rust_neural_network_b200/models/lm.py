"""Language-model wrappers used by the headline benchmark configurations.

`LoopedTransformerLM` = token `Embedding` (+ learned positions) -> `LoopedTransformer` trunk (a shared
block of `layers_per_block` pre-norm layers applied `loops` times with per-loop time conditioning,
rust-nn src/looped_transformer.rs:251-358) -> final LayerNorm -> LM head, trained with the fused
head+cross-entropy kernel pair. Weights are N(0, 0.02); compute is bf16 with fp32 master weights.
"""
from __future__ import annotations

import torch

from .. import nn
from ..ops import functional as F
from ..ops.transformer import lm_head_ce
from ..parallel.ddp import mark
from .looped_transformer import LoopedTransformer, _add_row


class LoopedTransformerLM(nn.Module):
    def __init__(self, vocab: int, d_model: int, heads: int, ff_dim: int, layers_per_block: int, loops: int,
                 max_seq: int, causal: bool = True, init_std: float = 0.02):
        init = nn.normal_init(init_std)
        self.vocab, self.d_model, self.max_seq = vocab, d_model, max_seq
        self.tok = nn.Embedding(vocab, d_model, std=init_std)
        self.pos = nn.Embedding(max_seq, d_model, std=init_std)
        # the trunk's own `embed` / `head` Linears are bypassed: tokens come from the embedding table
        self.core = LoopedTransformer(d_model, d_model, heads, ff_dim, d_model, loops, causal=causal,
                                      layers_per_block=layers_per_block, init=init)
        self.lm_head = nn.Linear(d_model, vocab, bias=True, init=init)

    def parameters(self):
        c = self.core
        return (self.tok.parameters() + self.pos.parameters() + c.block.parameters() + c.ln_final.parameters()
                + c.time_proj.parameters() + self.lm_head.parameters())

    def hidden(self, ids):
        B, S = ids.shape
        h = self.tok(ids)                                              # [B, S, d]
        pos = F.embedding(torch.arange(S, device=ids.device), self.pos.weight, self.compute_dtype)
        h = _add_rows(h, pos)
        h, _ = self.core.trunk(h)
        return self.core.ln_final(mark(h, 1))

    def dp_groups(self):
        """Parameter groups in the order their gradients complete LAST -> FIRST during backward (group 1 is final as
        soon as backward has passed the trunk's output; the shared block accumulates over all loops)."""
        c = self.core
        return [self.tok.parameters() + self.pos.parameters() + c.block.parameters() + c.time_proj.parameters(),
                c.ln_final.parameters() + self.lm_head.parameters()]

    def forward(self, ids):
        return self.lm_head(self.hidden(ids))

    def loss(self, ids, labels):
        """Mean next-token cross-entropy (labels are given explicitly; shape of `ids`)."""
        return lm_head_ce(self.hidden(ids), self.lm_head.weight, self.lm_head.bias, labels)


class _AddRowsFn(torch.autograd.Function):
    """a [B, S, d] + p [S, d] (broadcast over batch); dp = sum over batch."""

    @staticmethod
    def forward(ctx, a, p):
        from ..ops import kernels as K
        return K.binary(a, p, "add")

    @staticmethod
    def backward(ctx, g):
        from ..ops import kernels as K
        B = g.shape[0]
        return g, K.colsum(g.reshape(B, -1)).view(g.shape[1:])


def _add_rows(a, p):
    return _AddRowsFn.apply(a, p)
