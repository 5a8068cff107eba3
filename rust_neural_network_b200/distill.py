"""Knowledge distillation (rust-nn src/distill.rs): `DistillConfig`, `Distiller`, `ProgressiveDistiller`.

Loss: alpha * CE(student, labels) + beta * T^2 * soft term between the temperature-T softmaxes of
student and teacher. The reference's soft term is a squared difference whose inputs are detached,
so it carries no gradient (src/distill.rs:402-431); here the default `soft="kl"` is the real
KL(teacher || student) with a gradient, and `soft="mse"` is the differentiable squared difference.
The student generator follows src/distill.rs:165-203 (half the teacher's first hidden width, half
its depth, at least 16 / 1).
"""
from __future__ import annotations

import dataclasses
from typing import List

import torch

from . import nn
from .loss import CrossEntropyLoss
from .optim import Adam
from .train import SimpleDataLoader


@dataclasses.dataclass
class DistillConfig:
    temperature: float = 4.0
    alpha: float = 0.3
    beta: float = 0.5
    gamma: float = 0.2
    epochs: int = 20
    lr: float = 1e-3
    batch_size: int = 32
    student_hidden: int = 0
    student_layers: int = 0
    quantize_output: bool = False
    soft: str = "kl"
    verbose: bool = False

    def with_temperature(self, t: float):
        self.temperature = t; return self

    def with_weights(self, alpha: float, beta: float, gamma: float):
        self.alpha, self.beta, self.gamma = alpha, beta, gamma; return self

    def auto_student(self):
        self.student_hidden = 0; self.student_layers = 0; return self

    def quantize(self):
        self.quantize_output = True; return self


@dataclasses.dataclass
class DistillResult:
    student: nn.Sequential
    teacher_accuracy: float
    student_accuracy: float
    compression_ratio: float
    final_loss: float
    loss_history: List[float]


def softmax_temp(logits, t: float):
    return torch.softmax(logits.float() / t, -1)


def compute_accuracy(model, inputs, targets) -> float:
    with torch.no_grad():
        logits = model(inputs.to(model.device)) if hasattr(model, "device") else model(inputs)
    if logits.dim() < 2:
        return 0.0
    pred = logits.float().argmax(-1).cpu()
    t = targets.cpu()
    tgt = t.float().argmax(-1) if (t.dim() == 2 and t.shape[-1] == logits.shape[-1]) else t.reshape(t.shape[0], -1)[:, 0].long()
    return float((pred == tgt).float().mean())


class Distiller:
    def __init__(self, teacher, config: DistillConfig = None):
        self.teacher, self.config = teacher, config or DistillConfig()

    def generate_student(self, input_dim: int, output_dim: int) -> nn.Sequential:
        shapes = [tuple(p.shape) for p in self.teacher.parameters() if p.dim() == 2]
        teacher_hidden = shapes[0][0] if shapes else 64
        hidden = self.config.student_hidden or max(teacher_hidden // 2, 16)
        layers = self.config.student_layers or max(len(shapes) // 2, 1)
        model, prev = nn.Sequential(), input_dim
        for i in range(layers):
            out = output_dim if i == layers - 1 else hidden
            model.add(nn.Linear(prev, out))
            if i < layers - 1:
                model.add(nn.ReLU())
            prev = out
        return model

    def distill(self, inputs, targets, input_dim: int, output_dim: int) -> DistillResult:
        cfg = self.config
        dev = self.teacher.device if hasattr(self.teacher, "device") else torch.device("cpu")
        student = self.generate_student(input_dim, output_dim).to_device(dev)
        n_t = sum(p.numel() for p in self.teacher.parameters())
        n_s = sum(p.numel() for p in student.parameters())
        opt = Adam(student.parameters(), lr=cfg.lr)
        ce, T = CrossEntropyLoss(), cfg.temperature
        history = []
        for epoch in range(cfg.epochs):
            tot, nb = None, 0
            for xb, yb in SimpleDataLoader(inputs, targets, cfg.batch_size):
                xb, yb = xb.to(dev), yb.to(dev)
                opt.zero_grad()
                with torch.no_grad():
                    tp = softmax_temp(self.teacher(xb), T)
                sl = student(xb)
                hard = ce(sl, yb)
                if cfg.soft == "kl":
                    soft = (tp * (torch.log(tp.clamp_min(1e-12)) - torch.log_softmax(sl.float() / T, -1))).sum(-1).mean()
                else:
                    soft = ((softmax_temp(sl, T) - tp) ** 2).sum()
                loss = cfg.alpha * hard + cfg.beta * T * T * soft
                loss.backward()
                opt.step()
                tot = loss.detach() if tot is None else tot + loss.detach()
                nb += 1
            history.append(float(tot) / nb if nb else 0.0)
            if cfg.verbose and ((epoch + 1) % 5 == 0 or epoch == 0):
                print(f"  Distill epoch {epoch + 1}: loss = {history[-1]:.4f}")
        return DistillResult(student, compute_accuracy(self.teacher, inputs, targets), compute_accuracy(student, inputs, targets),
                             n_t / max(n_s, 1), history[-1] if history else 0.0, history)


class ProgressiveDistiller:
    """Repeated distillation: each round's student becomes the next round's teacher (src/distill.rs:309-345)."""

    def __init__(self, config: DistillConfig, rounds: int):
        self.config, self.rounds = config, rounds

    def distill(self, initial_teacher, inputs, targets, input_dim: int, output_dim: int) -> List[DistillResult]:
        results, teacher = [], initial_teacher
        for _ in range(self.rounds):
            r = Distiller(teacher, dataclasses.replace(self.config)).distill(inputs, targets, input_dim, output_dim)
            results.append(r)
            teacher = r.student
        return results


from ._compat import install as _install  # noqa: E402

_install(globals())
