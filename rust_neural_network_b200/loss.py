"""Losses (rust-nn src/loss.rs:11-82) on the fused loss kernels.

Reductions follow the reference: `MSELoss` is the SUM of squared errors by default
(src/loss.rs:20-26; pass `reduction="mean"` for the usual mean), `CrossEntropyLoss` is the mean over
the batch, the others are means over elements.
"""
from __future__ import annotations

import torch

from .ops import functional as F


from ._compat import NewMixin as _NewMixin  # noqa: E402

class Loss(_NewMixin):
    def forward(self, pred, target):
        raise NotImplementedError

    def __call__(self, pred, target):
        return self.forward(pred, target)


class MSELoss(Loss):
    def __init__(self, reduction: str = "sum"):
        self.reduction = reduction

    def forward(self, pred, target):
        return F.pointwise_loss(pred, target, "mse", 1.0, self.reduction)


class CrossEntropyLoss(Loss):
    """Logits + integer labels, or logits + one-hot / soft targets (the reference's only form,
    src/tensor.rs:464-496); mean over rows."""

    def forward(self, pred, target):
        return F.cross_entropy(pred, target)


class BCELoss(Loss):
    def forward(self, pred, target):
        return F.pointwise_loss(pred, target, "bce", 1.0, "mean")


class BCEWithLogitsLoss(Loss):
    def forward(self, pred, target):
        return F.pointwise_loss(pred, target, "bce_logits", 1.0, "mean")


class L1Loss(Loss):
    def forward(self, pred, target):
        return F.pointwise_loss(pred, target, "l1", 1.0, "mean")


class HuberLoss(Loss):
    def __init__(self, delta: float = 1.0):
        self.delta = delta

    def forward(self, pred, target):
        return F.pointwise_loss(pred, target, "huber", self.delta, "mean")


from ._compat import install as _install  # noqa: E402

_install(globals())
