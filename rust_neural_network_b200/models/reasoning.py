"""Reasoning wrappers (rust-nn src/reasoning.rs): `ChainOfThought`, `TreeOfThoughts`, `SwiReasoning`,
`MarkovianRSA`. Same constructors, defaults and parameter order as the reference; the thought
layers are fused Linear(+ReLU) GEMMs, beam scoring keeps all candidates on the device and reads
the scores back once per step (the reference reads one scalar per candidate).
"""
from __future__ import annotations

import torch

from .. import nn
from .looped_transformer import _add


def _thought(hidden):
    return nn.Sequential(nn.Linear(hidden, hidden), nn.ReLU(), nn.Linear(hidden, hidden))


class ChainOfThought(nn.Module):
    """state <- state + thought(state), `num_steps` times (residual on by default, src/reasoning.rs:133-193)."""

    def __init__(self, hidden_dim: int, num_steps: int):
        self.thought_layer = _thought(hidden_dim)
        self.num_steps, self.use_residual = num_steps, True

    def with_residual(self, use_residual: bool):
        self.use_residual = use_residual
        return self

    def forward(self, x):
        s = x
        for _ in range(self.num_steps):
            nxt = self.thought_layer(s)
            s = _add(s, nxt) if self.use_residual else nxt
        return s

    def parameters(self):
        return self.thought_layer.parameters()


class TreeOfThoughts(nn.Module):
    """Beam search over thought-layer expansions: every beam spawns `branching_factor` candidates
    (branches > 0 get uniform exploration noise, detached as in the reference), the evaluator's mean
    output scores them, the best `beam_width` survive (src/reasoning.rs:195-297)."""

    def __init__(self, hidden_dim: int, num_steps: int, branching_factor: int, beam_width: int, seed: int = 0):
        self.thought_layer = _thought(hidden_dim)
        self.evaluator = nn.Linear(hidden_dim, 1)
        self.num_steps, self.branching_factor, self.beam_width = num_steps, branching_factor, beam_width
        self.exploration_noise = 0.1
        self._gen = torch.Generator().manual_seed(seed)

    def with_exploration_noise(self, noise: float):
        self.exploration_noise = noise
        return self

    def score(self, state) -> torch.Tensor:
        return self.evaluator(state).float().mean()

    def forward(self, x):
        beams = [x]
        for _ in range(self.num_steps):
            cands = []
            for beam in beams:
                for br in range(self.branching_factor):
                    c = self.thought_layer(beam)
                    if self.exploration_noise > 0 and br > 0:
                        n = (torch.rand(c.shape, generator=self._gen) * 2 - 1) * self.exploration_noise
                        c = (c.detach() + n.to(c.device, c.dtype)).requires_grad_(c.requires_grad)
                    cands.append(c)
            scores = torch.stack([self.score(c).detach() for c in cands]).cpu().tolist()      # one read-back per step
            order = sorted(range(len(cands)), key=lambda i: -scores[i])[: self.beam_width]
            beams = [cands[i] for i in order]
        return beams[0] if beams else x

    def parameters(self):
        return self.thought_layer.parameters() + self.evaluator.parameters()


class SwiReasoning(nn.Module):
    """Four thinking steps that switch between a latent and an explicit layer whenever the confidence
    proxy mean|h| drops below the threshold (at most `max_switch_count` switches, src/reasoning.rs:14-79)."""

    def __init__(self, hidden_dim: int, max_switch_count: int, entropy_threshold: float):
        self.latent_layer = nn.Sequential(nn.Linear(hidden_dim, hidden_dim))
        self.explicit_layer = nn.Sequential(nn.Linear(hidden_dim, hidden_dim))
        self.max_switch_count, self.entropy_threshold = max_switch_count, entropy_threshold

    def calculate_confidence(self, h) -> float:
        return float(h.detach().float().abs().mean())

    def forward(self, x):
        s, switches, latent = x, 0, True
        for _ in range(4):
            if self.calculate_confidence(s) < self.entropy_threshold and switches < self.max_switch_count:
                latent = not latent
                switches += 1
            s = self.latent_layer(s) if latent else self.explicit_layer(s)
        return s

    def parameters(self):
        return self.latent_layer.parameters() + self.explicit_layer.parameters()


class MarkovianRSA(nn.Module):
    """Sum of `num_parallel_traces` copies of the input; the aggregation Linear exists (and is a
    parameter) but is not applied, exactly as in the reference (src/reasoning.rs:81-131)."""

    def __init__(self, hidden_dim: int, num_parallel_traces: int, chunk_duration: int):
        self.num_parallel_traces, self.chunk_duration = num_parallel_traces, chunk_duration
        self.aggregation_layer = nn.Linear(hidden_dim * num_parallel_traces, hidden_dim)

    def forward(self, x):
        out = x
        for _ in range(1, self.num_parallel_traces):
            out = _add(out, x)
        return out

    def parameters(self):
        return self.aggregation_layer.parameters()


from .._compat import install as _install  # noqa: E402

_install(globals())
