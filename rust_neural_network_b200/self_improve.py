"""Self-improvement loop (rust-nn src/self_improve.rs): a `Critic` scores the model's own output and,
when the reward reaches the threshold, the output is back-propagated with a gradient equal to the
reward in every element, followed by an optimizer step (src/self_improve.rs:52-74)."""
from __future__ import annotations

import torch


class Critic:
    """Interface: `evaluate(input, output) -> float`."""

    def evaluate(self, inp, out) -> float:
        raise NotImplementedError


class SelfImprover:
    def __init__(self, model, optimizer, critic: Critic, reward_threshold: float):
        self.model, self.optimizer, self.critic, self.reward_threshold = model, optimizer, critic, reward_threshold

    def self_train_step(self, unlabeled_input) -> float:
        self.optimizer.zero_grad()
        out = self.model(unlabeled_input)
        reward = float(self.critic.evaluate(unlabeled_input, out))
        if reward >= self.reward_threshold:
            out.backward(torch.full_like(out, reward))
            self.optimizer.step()
        return reward

    def self_train_epoch(self, inputs) -> float:
        total, n = 0.0, 0
        for x in inputs:
            total += self.self_train_step(x)
            n += 1
        return total / n if n else 0.0


from ._compat import install as _install  # noqa: E402

_install(globals())
