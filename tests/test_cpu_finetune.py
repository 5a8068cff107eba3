"""finetune.py, one test per behaviour of rust-nn src/finetune.rs:465-690: the LoRA adapter (shape, zero start, merge,
parameter count, construction from a layer), the three learning-rate schedules, the trainer with and without gradient
accumulation, the config builder and gradient clipping."""
import torch

from rust_neural_network_b200 import finetune as FT
from rust_neural_network_b200 import loss as L
from rust_neural_network_b200 import nn
from rust_neural_network_b200.optim import Adam
from rust_neural_network_b200.train import SimpleDataLoader


def test_lora_forward_shape():
    y = FT.LoraAdapter.new(64, 32, 8, 16.0).forward(torch.randn(4, 64))
    assert tuple(y.shape) == (4, 32)


def test_lora_starts_with_a_zero_update():
    assert float(FT.LoraAdapter.new(8, 4, 2, 4.0).weight_delta().abs().max()) < 1e-6


def test_lora_merge_matches_forward():
    torch.manual_seed(0)
    lora = FT.LoraAdapter.new(8, 4, 2, 4.0)
    lora.lora_b.data.fill_(0.1)
    x = torch.randn(2, 8)
    y = lora.forward(x)
    y_merged = x @ lora.merge().t() + (lora.bias if lora.bias is not None else 0.0)
    assert float((y.float() - y_merged).abs().max()) < 1e-4
    assert abs(lora.scale - 2.0) < 1e-9


def test_lora_trains_far_fewer_parameters():
    lora = FT.LoraAdapter.new(256, 256, 8, 16.0)
    assert sum(p.numel() for p in lora.trainable_parameters()) == 2 * 8 * 256
    assert sum(p.numel() for p in lora.trainable_parameters()) < 256 * 256 // 10
    assert not lora.frozen_weight.requires_grad


def test_lr_schedule_constant():
    s = FT.LrSchedule.Constant()
    assert abs(s.lr(0) - 0.001) < 1e-6 and abs(s.lr(1000) - 0.001) < 1e-6


def test_lr_schedule_warmup():
    s = FT.LrSchedule.Warmup(100, 0.01)
    assert s.lr(0) < 0.001 and abs(s.lr(100) - 0.01) < 1e-6 and abs(s.lr(500) - 0.01) < 1e-6
    assert abs(s.lr(50) - 0.005) < 1e-9


def test_lr_schedule_cosine_with_warmup():
    s = FT.LrSchedule.CosineWithWarmup(10, 100, 0.01, 0.001)
    assert s.lr(5) < s.lr(10) and abs(s.lr(10) - 0.01) < 1e-6
    assert s.lr(50) < 0.01 and s.lr(99) > 0.0009
    assert abs(s.lr(55) - 0.0055) < 1e-6                                     # half way down the cosine


def _fit(accum, clip, epochs, schedule, batch, rows, out, log_every=100):
    torch.manual_seed(1)
    model = nn.Sequential().add(nn.Linear(4, 16)).add(nn.ReLU()).add(nn.Linear(16, out))
    opt = Adam(model.parameters(), lr=0.01)
    cfg = FT.FastTrainConfig(epochs=epochs, micro_batch_size=batch, grad_accum_steps=accum, base_lr=0.01, lr_schedule=schedule,
                             grad_clip=clip, log_every=log_every)
    tr = FT.FastTrainer(model, cfg)
    hist = tr.fit(SimpleDataLoader(torch.randn(rows, 4), torch.randn(rows, out), batch), opt, L.MSELoss())
    return tr, hist


def test_fast_trainer_trains():
    tr, hist = _fit(1, 1.0, 5, FT.LrSchedule.Warmup(2, 0.01), 16, 64, 1, log_every=5)
    assert tr.total_steps() == 5 * 4 and len(hist) == 4                     # a history point every `log_every` steps
    assert hist[-1].loss < hist[0].loss * 1.5 and all(h.loss == h.loss for h in hist)
    _, quiet = _fit(1, 1.0, 1, FT.LrSchedule.Constant(), 16, 64, 1)
    assert quiet == []                                                      # fewer steps than `log_every`: nothing recorded


def test_fast_trainer_gradient_accumulation():
    tr, _ = _fit(4, 0.0, 2, FT.LrSchedule.Constant(), 8, 32, 2)
    assert tr.total_steps() > 0
    assert tr.total_steps() == 2                                             # 4 micro-batches of 8 = one optimizer step per epoch


def test_config_builder():
    cfg = FT.FastTrainConfig().with_lora(16, 32.0).with_accum(8).with_grad_clip(5.0)
    assert cfg.use_lora and cfg.lora_rank == 16 and cfg.grad_accum_steps == 8 and cfg.grad_clip == 5.0
    assert cfg.effective_batch_size() == 32 * 8


def test_lora_from_linear_freezes_the_original_weight():
    layer = nn.Linear(32, 16)
    ad = FT.LoraAdapter.from_linear(layer, 4, 8.0)
    assert (ad.rank, ad.in_features, ad.out_features) == (4, 32, 16)
    assert torch.equal(ad.frozen_weight.detach(), layer.weight.detach())
    x = torch.randn(3, 32)
    assert torch.allclose(ad.forward(x).float(), layer(x).float(), atol=1e-5)      # zero update at the start


def test_clip_grad_norm():
    t = torch.tensor([3.0, 4.0], requires_grad=True)
    t.grad = torch.full((2,), 10.0)
    FT.clip_grad_norm([t], 1.0)
    assert float(t.grad.norm()) <= 1.01
