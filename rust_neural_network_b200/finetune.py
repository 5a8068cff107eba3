"""Fine-tuning utilities (rust-nn src/finetune.rs): `LoraAdapter`, `LrSchedule`, `FastTrainConfig`,
`FastTrainer`, `TrainPoint`.

LoRA: y = x W^T + b + (alpha/r) (x A^T) B^T with W frozen, A ~ U(-0.01, 0.01), B = 0
(src/finetune.rs:61-151). The low-rank path runs as two GEMMs whose second one adds the frozen
path's output through the kernel's residual epilogue, so the adapter costs no extra pass over y.
`FastTrainer.fit`: gradient accumulation over micro-batches, global-norm clipping on the device
(no host sync), and - unlike the reference, which computes the scheduled LR but never applies it
(src/finetune.rs:368-370) - the schedule really drives the optimizer.
"""
from __future__ import annotations

import dataclasses
import math
import time
from typing import List, Optional

import torch

from . import nn
from .ops import functional as F


class LoraAdapter(nn.Module):
    def __init__(self, in_features: int, out_features: int, rank: int, alpha: float):
        self.in_features, self.out_features, self.rank, self.alpha = in_features, out_features, rank, alpha
        self.frozen_weight = torch.nn.Parameter(nn.he_normal((out_features, in_features)), requires_grad=False)
        self.lora_a = nn._param(torch.rand(rank, in_features) * 0.02 - 0.01)
        self.lora_b = nn._param(torch.zeros(out_features, rank))
        self.bias: Optional[torch.Tensor] = torch.nn.Parameter(torch.zeros(out_features), requires_grad=False)

    @staticmethod
    def new(in_features, out_features, rank, alpha) -> "LoraAdapter":
        return LoraAdapter(in_features, out_features, rank, alpha)

    @staticmethod
    def from_linear(layer: nn.Linear, rank: int, alpha: float) -> "LoraAdapter":
        ad = LoraAdapter(layer.in_features, layer.out_features, rank, alpha)
        ad.frozen_weight = torch.nn.Parameter(layer.weight.detach().clone(), requires_grad=False)
        ad.bias = torch.nn.Parameter(layer.bias.detach().clone(), requires_grad=False) if layer.bias is not None else None
        dev = layer.weight.device
        for t in (ad.lora_a, ad.lora_b):
            t.data = t.data.to(dev)
        return ad

    @property
    def scale(self) -> float:
        return self.alpha / self.rank

    def forward(self, x):
        base = F.linear(x, self.frozen_weight, self.bias, "none", None)                 # frozen path
        low = F.linear(x, self.lora_a, None, "none", None)                              # x A^T          [.., r]
        return F.linear(low * self.scale, self.lora_b, None, "none", base)              # (..) B^T + base (residual epilogue)

    def trainable_parameters(self):
        return [self.lora_a, self.lora_b]

    def parameters(self):
        return self.trainable_parameters()

    def weight_delta(self) -> torch.Tensor:
        return (self.lora_b.detach() @ self.lora_a.detach()) * self.scale

    def merge(self) -> torch.Tensor:
        return self.frozen_weight.detach() + self.weight_delta()

    def own_parameters(self):
        return [self.lora_a, self.lora_b]


class LrSchedule:
    """`Constant` (returns 0.001, as the reference), `Warmup{warmup_steps, base_lr}`,
    `CosineWithWarmup{warmup_steps, total_steps, base_lr, min_lr}` (src/finetune.rs:157-203)."""

    def __init__(self, kind="constant", warmup_steps=0, total_steps=0, base_lr=1e-3, min_lr=0.0):
        self.kind, self.warmup_steps, self.total_steps, self.base_lr, self.min_lr = kind, warmup_steps, total_steps, base_lr, min_lr

    @staticmethod
    def Constant(): return LrSchedule("constant")
    @staticmethod
    def Warmup(warmup_steps, base_lr): return LrSchedule("warmup", warmup_steps, 0, base_lr)
    @staticmethod
    def CosineWithWarmup(warmup_steps, total_steps, base_lr, min_lr): return LrSchedule("cosine", warmup_steps, total_steps, base_lr, min_lr)

    def lr(self, step: int) -> float:
        if self.kind == "constant":
            return 0.001
        if step < self.warmup_steps:
            return self.base_lr * (step / self.warmup_steps)
        if self.kind == "warmup":
            return self.base_lr
        progress = (step - self.warmup_steps) / max(self.total_steps - self.warmup_steps, 1)
        return self.min_lr + (self.base_lr - self.min_lr) * 0.5 * (1.0 + math.cos(math.pi * progress))


@dataclasses.dataclass
class FastTrainConfig:
    epochs: int = 10
    micro_batch_size: int = 32
    grad_accum_steps: int = 1
    base_lr: float = 1e-3
    lr_schedule: LrSchedule = dataclasses.field(default_factory=lambda: LrSchedule.CosineWithWarmup(100, 1000, 1e-3, 1e-4))
    grad_clip: float = 1.0
    use_lora: bool = False
    lora_rank: int = 8
    lora_alpha: float = 16.0
    log_every: int = 10
    apply_schedule: bool = True      # the reference never applies the scheduled LR; set False for that behaviour
    verbose: bool = False

    def effective_batch_size(self) -> int:
        return self.micro_batch_size * self.grad_accum_steps

    def with_lora(self, rank: int, alpha: float):
        self.use_lora, self.lora_rank, self.lora_alpha = True, rank, alpha
        return self

    def with_accum(self, steps: int):
        self.grad_accum_steps = steps
        return self

    def with_grad_clip(self, clip: float):
        self.grad_clip = clip
        return self


@dataclasses.dataclass
class TrainPoint:
    epoch: int
    step: int
    loss: float
    lr: float
    elapsed_secs: float


def clip_grad_norm(params, max_norm: float) -> float:
    """Global-norm clipping of `.grad` tensors in place (rust-nn src/finetune.rs / src/distributed.rs:507-523)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0.0
    total = torch.sqrt(sum((g.float() ** 2).sum() for g in grads))
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return float(total)


class FastTrainer:
    def __init__(self, model, config: Optional[FastTrainConfig] = None, logger=None):
        """`logger`: a `utils.metrics.MetricsLogger`; every recorded `TrainPoint` is also appended to it as one JSON line."""
        self._model = model
        self.logger = logger
        self.config = config or FastTrainConfig()
        self._history: List[TrainPoint] = []
        self._total_steps = 0

    @staticmethod
    def new_lora(model, rank: int, alpha: float, config: Optional[FastTrainConfig] = None) -> "FastTrainer":
        cfg = config or FastTrainConfig()
        cfg.with_lora(rank, alpha)
        return FastTrainer(model, cfg)

    def fit(self, loader, optimizer, loss_fn) -> List[TrainPoint]:
        cfg = self.config
        start = time.time()
        step = 0
        dev = self._model.device
        for epoch in range(cfg.epochs):
            accum, losses = 0, []
            optimizer.zero_grad()

            def do_step():
                nonlocal step
                if cfg.grad_clip > 0:
                    if hasattr(optimizer, "clip_grad_norm"):
                        optimizer.clip_grad_norm(cfg.grad_clip)
                    else:
                        clip_grad_norm(self._model.parameters(), cfg.grad_clip)
                lr = cfg.lr_schedule.lr(step)
                if cfg.apply_schedule and hasattr(optimizer, "set_lr") and cfg.lr_schedule.kind != "constant":
                    optimizer.set_lr(max(lr, 1e-12))
                optimizer.step()
                optimizer.zero_grad()
                step += 1
                self._total_steps += 1
                return lr

            for x, y in loader:
                x, y = _unwrap(x), _unwrap(y)
                x = x.to(dev, non_blocking=True); y = y.to(dev, non_blocking=True)
                loss = loss_fn(self._model(x), y)
                loss.backward()
                losses.append(loss.detach().float() / max(x.shape[0], 1))
                accum += 1
                if accum >= cfg.grad_accum_steps:
                    lr = do_step()
                    accum = 0
                    if step % cfg.log_every == 0:
                        elapsed = time.time() - start
                        pt = TrainPoint(epoch, step, float(torch.stack(losses).mean()), lr, elapsed)
                        self._history.append(pt)
                        if self.logger is not None:
                            self.logger.log(step, epoch=epoch, loss=pt.loss, lr=pt.lr, steps_per_s=step / max(elapsed, 1e-9))
                        if cfg.verbose:
                            print(f"  Epoch {epoch + 1} Step {step}: loss={pt.loss:.4f} lr={pt.lr:.6f} ({step / max(elapsed, 1e-9):.1f} steps/s)")
            if accum > 0:
                do_step()
            if cfg.verbose and losses:
                print(f"  Epoch {epoch + 1} done: avg_loss={float(torch.stack(losses).mean()):.4f} ({time.time() - start:.1f}s)")
        return list(self._history)

    def history(self) -> List[TrainPoint]:
        return self._history

    def total_steps(self) -> int:
        return self._total_steps

    def model(self):
        return self._model


from ._compat import install as _install, unwrap as _unwrap  # noqa: E402

_install(globals())
