"""DDPM (rust-nn src/diffusion.rs): `NoiseSchedule` (linear 1e-4..0.02 / cosine), `sinusoidal_embedding`,
`DenoiseNet` (time_proj Linear-SiLU-Linear added to the input, net Linear-SiLU-Linear-SiLU-Linear),
`DDPM` with `q_sample`, `predict_noise`, `train_batch`, `sample`.

The reference draws its "noise" from U(-1, 1) (src/diffusion.rs:212,234,249); `noise="uniform"`
reproduces that, the default `noise="gaussian"` is the DDPM definition. Everything runs on the
model's device; the MLPs are the fused Linear+SiLU GEMM epilogues.
"""
from __future__ import annotations

import enum
import math

import torch

from .. import nn
from ..loss import MSELoss
from .looped_transformer import _add_row, sinusoidal_embedding   # re-exported: same definition as src/diffusion.rs:89-105


class ScheduleType(enum.Enum):
    Linear = 0
    Cosine = 1


class NoiseSchedule:
    def __init__(self, schedule: ScheduleType, timesteps: int):
        self.timesteps = timesteps
        if schedule == ScheduleType.Linear:
            b0, b1 = 1e-4, 0.02
            betas = [b0 + (b1 - b0) * i / max(timesteps - 1, 1) for i in range(timesteps)]
        else:
            f = lambda x: math.cos(x * math.pi / 2.0) ** 2
            betas = [min(1.0 - f((t + 1) / timesteps) / f(t / timesteps), 0.999) for t in range(timesteps)]
            if betas[0] < 1e-6:
                betas[0] = 1e-6
        self.betas = betas
        self.alphas = [1.0 - b for b in betas]
        acc, cum = 1.0, []
        for a in self.alphas:
            acc *= a
            cum.append(max(acc, 1e-12))
        self.alpha_cumprod = cum
        self.sqrt_alpha_cumprod = [math.sqrt(a) for a in cum]
        self.sqrt_one_minus_alpha_cumprod = [math.sqrt(1.0 - a) for a in cum]

    @staticmethod
    def new(schedule: ScheduleType, timesteps: int) -> "NoiseSchedule":
        return NoiseSchedule(schedule, timesteps)


class DenoiseNet(nn.Module):
    def __init__(self, data_dim: int, hidden_dim: int, time_embed_dim: int):
        self.data_dim, self.time_embed_dim = data_dim, time_embed_dim
        self.time_proj = nn.Sequential(nn.Linear(time_embed_dim, hidden_dim), nn.SiLU(), nn.Linear(hidden_dim, data_dim))
        self.net = nn.Sequential(nn.Linear(data_dim, hidden_dim), nn.SiLU(), nn.Linear(hidden_dim, hidden_dim), nn.SiLU(),
                                 nn.Linear(hidden_dim, data_dim))

    def predict(self, x_t, t: int):
        temb = sinusoidal_embedding(float(t), self.time_embed_dim, x_t.device).to(x_t.dtype)
        tcond = self.time_proj(temb).reshape(self.data_dim)
        return self.net(_add_row(x_t, tcond))

    def forward(self, x):
        return self.net(x)

    def parameters(self):
        return self.time_proj.parameters() + self.net.parameters()


class DDPM(nn.Module):
    def __init__(self, data_dim: int, hidden_dim: int, timesteps: int, schedule: ScheduleType = ScheduleType.Linear,
                 noise: str = "gaussian", seed: int = 0):
        self.data_dim = data_dim
        self.schedule = NoiseSchedule(schedule, timesteps)
        self.denoise = DenoiseNet(data_dim, hidden_dim, min(max(data_dim, 16), 128))
        self.noise_kind = noise
        self._gen = torch.Generator().manual_seed(seed)

    def _noise(self, shape, device, dtype):
        if self.noise_kind == "uniform":
            n = torch.rand(shape, generator=self._gen) * 2 - 1
        else:
            n = torch.randn(shape, generator=self._gen)
        return n.to(device=device, dtype=dtype)

    def q_sample(self, x_0, t: int, noise):
        return x_0 * self.schedule.sqrt_alpha_cumprod[t] + noise * self.schedule.sqrt_one_minus_alpha_cumprod[t]

    def predict_noise(self, x_t, t: int):
        return self.denoise.predict(x_t, t)

    def train_batch(self, optimizer, x_0) -> float:
        """One optimisation step at a random timestep; returns the mean squared error (sum / n_elems, as the reference)."""
        t = int(torch.randint(0, self.schedule.timesteps, (1,), generator=self._gen))
        noise = self._noise(x_0.shape, x_0.device, x_0.dtype)
        x_t = self.q_sample(x_0.detach(), t, noise)
        optimizer.zero_grad()
        loss = MSELoss("sum")(self.predict_noise(x_t, t), noise)
        loss.backward()
        optimizer.step()
        return float(loss.detach()) / x_0.numel()

    @torch.no_grad()
    def sample(self, batch_size: int, device=None):
        device = device or self.denoise.device
        dtype = self.denoise.compute_dtype
        x = self._noise((batch_size, self.data_dim), device, dtype)
        s = self.schedule
        for t in reversed(range(s.timesteps)):
            pn = self.predict_noise(x, t)
            mean = (x - pn * (s.betas[t] / math.sqrt(1.0 - s.alpha_cumprod[t]))) / math.sqrt(s.alphas[t])
            x = mean + math.sqrt(s.betas[t]) * self._noise(x.shape, device, dtype) if t > 0 else mean
        return x

    def forward(self, x):
        return self.denoise(x)

    def parameters(self):
        return self.denoise.parameters()


from .._compat import install as _install  # noqa: E402

_install(globals())
