"""Model-compression toolkit (rust-nn src/compression.rs): `SharedWeights`, `SparseMatrix` (CSR),
`LayerDropper`, `KnowledgeTransfer`, `CompressedEmbedding`, `MixedSparsity`, `ProgressiveShrinking`,
`StructuredPruner`, `CompressionStrategy`, `CompressionRecipe`, `automl_search`.

Dense products go through this package's GEMM (`SharedWeights`, `CompressedEmbedding.reconstruct`,
`KnowledgeTransfer`), the CSR product is a CUDA kernel (one warp per row strip), and the magnitude
thresholds are order statistics computed on the device (`torch.kthvalue` / `sort`), not host sorts.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple

import torch

from . import nn
from .ops import functional as F
from .ops import quant_kernels as Q


class SharedWeights(nn.Module):
    """One Linear applied `num_passes` times (src/compression.rs:26-80)."""

    def __init__(self, in_features: int, out_features: int, num_passes: int):
        self.weight = nn._param(nn.he_normal((out_features, in_features)))
        self.bias = torch.nn.Parameter(torch.zeros(out_features), requires_grad=False)
        self.num_passes, self.in_features, self.out_features = num_passes, in_features, out_features

    def forward(self, x):
        h = x
        for _ in range(self.num_passes):
            h = F.linear(h, self.weight, self.bias, "none", None)
        return h

    def param_count(self) -> int:
        return self.weight.numel() + self.bias.numel()

    def compression_ratio(self) -> float:
        return float(self.num_passes)

    def parameters(self):
        return [self.weight, self.bias]


class SparseMatrix:
    """CSR matrix: `values` fp32, `col_indices` / `row_ptrs` int32 (device tensors)."""

    def __init__(self, values, col_indices, row_ptrs, rows: int, cols: int):
        self.values, self.col_indices, self.row_ptrs, self.rows, self.cols = values, col_indices, row_ptrs, rows, cols
        self.nnz = int(values.numel())

    @staticmethod
    def from_dense(tensor: torch.Tensor, threshold: float) -> "SparseMatrix":
        t = tensor.detach().float()
        rows = t.shape[0] if t.dim() >= 1 else 1
        cols = t.shape[1] if t.dim() >= 2 else t.numel()
        d = t.reshape(rows, cols)
        mask = d.abs() > threshold
        idx = mask.nonzero()                                   # row-major order = CSR order
        counts = mask.sum(-1)
        row_ptrs = torch.zeros(rows + 1, dtype=torch.int32, device=t.device)
        row_ptrs[1:] = counts.cumsum(0).to(torch.int32)
        return SparseMatrix(d[mask].contiguous(), idx[:, 1].to(torch.int32).contiguous(), row_ptrs, rows, cols)

    def spmm(self, b: torch.Tensor, n: int) -> torch.Tensor:
        """C[rows, n] = self * B with B [cols, n] (flat or 2-D)."""
        return Q.csr_spmm(self.values, self.col_indices, self.row_ptrs, b.reshape(self.cols, n).to(self.values.device), self.rows, n)

    def sparsity(self) -> float:
        return 1.0 - self.nnz / max(self.rows * self.cols, 1)

    def mem_bytes(self) -> int:
        return self.values.numel() * 4 + self.col_indices.numel() * 8 + self.row_ptrs.numel() * 8    # the reference's usize accounting

    def compression_ratio(self) -> float:
        return self.rows * self.cols * 4 / max(self.mem_bytes(), 1)

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self.rows, self.cols, dtype=torch.float32, device=self.values.device)
        r = torch.repeat_interleave(torch.arange(self.rows, device=out.device), (self.row_ptrs[1:] - self.row_ptrs[:-1]).long())
        out[r, self.col_indices.long()] = self.values
        return out


class LayerDropper:
    """Skips a layer whose output norm differs from its input norm by less than a threshold."""

    def __init__(self, num_layers: int, threshold: float):
        self.thresholds = [threshold] * num_layers
        self.skip_counts = [0] * num_layers
        self.total_count = 0

    def should_skip(self, layer_idx: int, before: torch.Tensor, after: torch.Tensor) -> bool:
        self.total_count += 1
        bn, an = float(before.detach().float().norm()), float(after.detach().float().norm())
        change = abs(an - bn) / max(bn, 1e-8)
        if change < self.thresholds[min(layer_idx, len(self.thresholds) - 1)]:
            self.skip_counts[min(layer_idx, len(self.skip_counts) - 1)] += 1
            return True
        return False

    def avg_skip_rate(self) -> float:
        if self.total_count == 0:
            return 0.0
        return sum(self.skip_counts) / (self.total_count * max(len(self.thresholds), 1))

    def estimated_speedup(self) -> float:
        return 1.0 / max(1.0 - self.avg_skip_rate(), 0.01)


class KnowledgeTransfer:
    """Feature-matching loss between a source and a target model through a learned projection."""

    def __init__(self, source, target, source_dim: int, target_dim: int):
        self.source, self.target = source, target
        self.projection = nn.Linear(source_dim, max(source_dim, target_dim), True)

    def transfer_loss_tensor(self, x) -> torch.Tensor:
        dev = x.device
        if self.projection.weight.device != dev:
            self.projection.to_device(dev)
        with torch.no_grad():
            s = self.source(x)
        t = self.target(x)
        d = self.projection(s).float() - t.float()
        return (d * d).mean()

    def transfer_loss(self, x) -> float:
        return float(self.transfer_loss_tensor(x).detach())


class CompressedEmbedding:
    """Low-rank embedding U[vocab, r] V[r, dim]. `from_table` follows the reference (random factors,
    src/compression.rs:304-319); `from_table_svd` fits the factors to the table."""

    def __init__(self, factor_u, factor_v):
        self.factor_u, self.factor_v = factor_u, factor_v
        self.vocab_size, self.rank = factor_u.shape
        self.embed_dim = factor_v.shape[1]

    @staticmethod
    def from_table(embedding: torch.Tensor, rank: int) -> "CompressedEmbedding":
        v, d = embedding.shape
        return CompressedEmbedding(torch.randn(v, rank, device=embedding.device), torch.randn(rank, d, device=embedding.device))

    @staticmethod
    def from_table_svd(embedding: torch.Tensor, rank: int) -> "CompressedEmbedding":
        u, s, vh = torch.linalg.svd(embedding.detach().float(), full_matrices=False)
        r = min(rank, s.numel())
        return CompressedEmbedding((u[:, :r] * s[:r]).contiguous(), vh[:r].contiguous())

    def lookup(self, token: int) -> torch.Tensor:
        return self.lookup_batch([token])

    def lookup_batch(self, tokens) -> torch.Tensor:
        ids = torch.as_tensor(tokens, dtype=torch.int64, device=self.factor_u.device)
        return F.matmul(F.embedding(ids, self.factor_u, torch.float32), self.factor_v)

    def reconstruct(self) -> torch.Tensor:
        return F.matmul(self.factor_u, self.factor_v)

    def compression_ratio(self) -> float:
        return self.vocab_size * self.embed_dim / (self.vocab_size * self.rank + self.rank * self.embed_dim)

    def mem_bytes(self) -> int:
        return (self.factor_u.numel() + self.factor_v.numel()) * 4


class MixedSparsity:
    """Per-parameter sparsity from a prune-half sensitivity probe (src/compression.rs:378-434)."""

    def __init__(self, layer_sparsity: List[float], sensitivity: List[float]):
        self.layer_sparsity, self.sensitivity = layer_sparsity, sensitivity

    @staticmethod
    def analyze(model, inputs, targets, loss_fn) -> "MixedSparsity":
        params = list(model.parameters())
        with torch.no_grad():
            base = float(loss_fn(model(inputs), targets))
            sens, sp = [], []
            for p in params:
                keep = p.data.clone()
                flat = p.data.abs().reshape(-1).float()
                thr = torch.sort(flat).values[flat.numel() // 2]
                p.data = torch.where(p.data.abs().float() < thr, torch.zeros_like(p.data), p.data)
                _bump(p)
                pruned = float(loss_fn(model(inputs), targets))
                p.data = keep
                _bump(p)
                inc = max(pruned - base, 0.0)
                sens.append(inc)
                sp.append(0.5 / (1.0 + inc * 10.0))
        avg = sum(sp) / max(len(sp), 1)
        scale = 0.5 / max(avg, 1e-8)
        return MixedSparsity([min(max(s * scale, 0.05), 0.9) for s in sp], sens)

    def sparsity_for_layer(self, layer_idx: int) -> float:
        return self.layer_sparsity[layer_idx] if 0 <= layer_idx < len(self.layer_sparsity) else 0.5


def _bump(p) -> None:
    """Invalidate a parameter's cached low-precision shadow after an in-place edit of `.data`."""
    if hasattr(p, "_lp_version"):
        p._lp_version = -1


class ProgressiveShrinking:
    def __init__(self, target_sparsity: float, total_steps: int, warmup_steps: int):
        self.target_sparsity, self.current_sparsity = target_sparsity, 0.0
        self.total_steps, self.current_step, self.warmup_steps = total_steps, 0, warmup_steps

    def step(self) -> float:
        self.current_step += 1
        if self.current_step <= self.warmup_steps:
            self.current_sparsity = 0.0
        elif self.current_step >= self.total_steps:
            self.current_sparsity = self.target_sparsity
        else:
            prog = (self.current_step - self.warmup_steps) / max(self.total_steps - self.warmup_steps, 1)
            self.current_sparsity = self.target_sparsity * prog
        return self.current_sparsity

    def apply_soft_prune(self, tensor: torch.Tensor) -> torch.Tensor:
        if self.current_sparsity <= 0.0:
            return tensor.clone()
        t = tensor.detach()
        n = t.numel()
        n_prune = int(n * self.current_sparsity)
        thr = torch.sort(t.abs().reshape(-1).float()).values[min(n_prune, n - 1)]
        return torch.where(t.abs().float() <= thr, torch.zeros_like(t), t)

    def is_done(self) -> bool:
        return self.current_step >= self.total_steps


class StructuredPruner:
    def __init__(self, prune_ratio: float, num_layers: int):
        self.prune_ratios = [prune_ratio] * num_layers

    @staticmethod
    def prune_channels(weight: torch.Tensor, prune_ratio: float) -> Tuple[torch.Tensor, List[int]]:
        """Keeps the output channels (rows) of largest L2 norm, in ascending norm order as the reference does."""
        w = weight.detach()
        out_f = w.shape[0]
        norms = w.float().reshape(out_f, -1).norm(dim=1)
        order = torch.sort(norms, stable=True).indices
        n_keep = min(max(int(round((1.0 - prune_ratio) * out_f)), 1), out_f)
        kept = order[out_f - n_keep:]
        return w[kept].clone(), kept.tolist()

    @staticmethod
    def prune_linear(layer: nn.Linear, prune_ratio: float) -> Tuple[nn.Linear, List[int]]:
        w, kept = StructuredPruner.prune_channels(layer.weight, prune_ratio)
        new = nn.Linear(layer.in_features, len(kept), bias=layer.bias is not None)
        new.weight = nn._param(w.float())
        if layer.bias is not None:
            new.bias = nn._param(layer.bias.detach()[torch.as_tensor(kept, device=layer.bias.device)].float().clone())
        return new, kept


@dataclasses.dataclass
class CompressionStrategy:
    """`kind` in {"none", "prune", "structured_prune", "low_rank", "quantize"} with its one parameter."""
    kind: str = "none"
    ratio: float = 0.0
    rank: int = 0
    bits: int = 0

    @staticmethod
    def None_(): return CompressionStrategy("none")
    @staticmethod
    def Prune(ratio: float): return CompressionStrategy("prune", ratio=ratio)
    @staticmethod
    def StructuredPrune(ratio: float): return CompressionStrategy("structured_prune", ratio=ratio)
    @staticmethod
    def LowRank(rank: int): return CompressionStrategy("low_rank", rank=rank)
    @staticmethod
    def Quantize(bits: int): return CompressionStrategy("quantize", bits=bits)

    def size_factor(self) -> float:
        if self.kind in ("prune", "structured_prune"):
            return 1.0 / (1.0 - self.ratio)
        if self.kind == "low_rank":
            return 4.0
        if self.kind == "quantize":
            return 32.0 / self.bits
        return 1.0


@dataclasses.dataclass
class CompressionRecipe:
    strategies: List[CompressionStrategy]
    compression_ratio: float
    accuracy_retention: float


def automl_search(model, inputs, targets, loss_fn, target_compression: float) -> CompressionRecipe:
    """The reference's greedy per-layer choice by a fixed quality score (src/compression.rs:641-725)."""
    params = list(model.parameters())
    n_layers = sum(1 for p in params if p.dim() == 2)
    with torch.no_grad():
        base = float(loss_fn(model(inputs), targets))
    cands = [CompressionStrategy.None_(), CompressionStrategy.Prune(0.3), CompressionStrategy.Prune(0.5), CompressionStrategy.Prune(0.7),
             CompressionStrategy.StructuredPrune(0.3), CompressionStrategy.Quantize(8), CompressionStrategy.Quantize(4)]
    strategies: List[CompressionStrategy] = []
    current = 1.0
    for i, p in enumerate(params):
        if p.dim() != 2:
            continue
        norm = float(p.detach().abs().float().mean())

        def score(s: CompressionStrategy) -> float:
            if s.kind == "none":
                return 1.0
            if s.kind == "prune":
                return (1.0 - s.ratio) * (norm / max(norm, 0.01))
            if s.kind == "structured_prune":
                return 1.0 - s.ratio * 0.5
            if s.kind == "quantize":
                return 1.0 - (32.0 / s.bits - 1.0) * 0.05
            return 0.8
        best, best_score = cands[0], -1.0
        for s in cands:                      # the last maximum wins, as Iterator::max_by
            sc = score(s)
            if sc >= best_score:
                best, best_score = s, sc
        strategies.append(best)
        current *= best.size_factor()
        if current >= target_compression and i >= n_layers // 2:
            strategies.extend(CompressionStrategy.None_() for _ in range(i + 1, len(params)))
            break
    return CompressionRecipe(strategies, current, 1.0 - base * 0.1)


from ._compat import install as _install  # noqa: E402

_install(globals())
