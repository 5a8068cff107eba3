"""Mamba and the DDPM, one test per behaviour of rust-nn tests/mamba_diffusion.rs:18-209."""
import math

import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.models.diffusion import DDPM, NoiseSchedule, ScheduleType
from rust_neural_network_b200.models.mamba import HybridMamba, Mamba, MambaBlock
from rust_neural_network_b200.optim import Adam


def test_mamba_block_preserves_shape():
    assert list(MambaBlock(8, 4, 2, 3)(torch.randn(2, 5, 8)).shape) == [2, 5, 8]


def test_mamba_block_is_differentiable():
    x = torch.tensor([math.sin(i * 0.07) for i in range(48)]).reshape(2, 4, 6).requires_grad_(True)
    MambaBlock(6, 3, 2, 3)(x).sum().backward()
    assert x.grad is not None and bool((x.grad.abs() > 0).any())


def test_mamba_block_is_causal():
    torch.manual_seed(0)
    block = MambaBlock(6, 3, 2, 3)
    x = torch.randn(1, 5, 6)
    x2 = x.clone()
    x2[0, 3:] += 1.0                                                # a change at t >= 3 must leave t < 3 as it was
    assert torch.allclose(block(x)[0, :3], block(x2)[0, :3], atol=1e-6)


def test_mamba_preserves_shape():
    assert list(Mamba(8, 4, 2, 3, 3)(torch.randn(2, 6, 8)).shape) == [2, 6, 8]


def test_mamba_exposes_its_parameters():
    assert len(Mamba(8, 4, 2, 3, 2).parameters()) > 10


def test_hybrid_mamba_preserves_shape():
    model = (HybridMamba(8).with_mamba(4, 2, 3).with_mamba(4, 2, 3)
             .with_layer(nn.Sequential().add(nn.Linear(8, 8)).add(nn.SiLU())).with_mamba(4, 2, 3))
    assert list(model(torch.randn(2, 5, 8)).shape) == [2, 5, 8]
    assert len(model.blocks) == 4


def test_mamba_training_reduces_the_copy_loss():
    torch.manual_seed(0)
    model = Mamba(4, 4, 2, 3, 2)
    opt = Adam(model.parameters(), lr=0.01)
    x = torch.tensor([0.3, -0.1, 0.5, 0.2, -0.4, 0.6, 0.1, -0.3, 0.2, 0.4, -0.5, 0.0]).reshape(1, 3, 4)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = ((model(x) - x) ** 2).sum()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0]


def test_linear_noise_schedule_is_valid():
    s = NoiseSchedule.new(ScheduleType.Linear, 100)
    betas, ac = list(s.betas), list(s.alpha_cumprod)
    assert len(betas) == 100 and all(0.0 <= float(b) < 1.0 for b in betas)
    assert all(float(b) <= float(a) + 1e-6 and 0.0 < float(a) <= 1.0 for a, b in zip(ac, ac[1:]))
    assert abs(float(ac[0]) - 1.0) < 1e-3


def test_cosine_noise_schedule_is_valid():
    s = NoiseSchedule.new(ScheduleType.Cosine, 50)
    assert all(0.0 <= float(b) < 1.0 for b in s.betas)
    assert float(s.alpha_cumprod[0]) > 0.99 and float(s.alpha_cumprod[49]) < float(s.alpha_cumprod[0])


def test_q_sample_endpoints():
    ddpm = DDPM(3, 16, 100, ScheduleType.Linear)
    x0, noise = torch.tensor([[1.0, 2.0, 3.0]]), torch.zeros(1, 3)
    assert abs(float(ddpm.q_sample(x0, 0, noise)[0, 0]) - 1.0) < 0.05       # alpha_bar ~ 1: x_t ~ x_0
    xt = ddpm.q_sample(x0, 99, noise)                                        # no noise: sqrt(alpha_bar) * x_0
    assert abs(float(xt[0, 0])) < 1.0
    assert torch.allclose(xt, math.sqrt(float(ddpm.schedule.alpha_cumprod[99])) * x0, atol=1e-6)


def test_ddpm_training_reduces_the_loss():
    torch.manual_seed(0)
    ddpm = DDPM(4, 32, 50, ScheduleType.Linear)
    opt = Adam(ddpm.parameters(), lr=0.01)
    x0 = torch.randn(8, 4)
    losses = [ddpm.train_batch(opt, x0) for _ in range(40)]
    assert sum(losses[-5:]) / 5 < sum(losses[:5]) / 5


def test_ddpm_sample_shape():
    s = DDPM(4, 16, 30, ScheduleType.Linear).sample(5)
    assert list(s.shape) == [5, 4] and bool(torch.isfinite(s).all())


def test_predict_noise_preserves_shape():
    assert list(DDPM(6, 16, 20, ScheduleType.Linear).predict_noise(torch.randn(3, 6), 5).shape) == [3, 6]
