"""distill.py, one test per behaviour of rust-nn src/distill.rs:400-560: the generated student is smaller than its
teacher, the config builder, a distillation run with its loss history, the softened softmax, accuracy, the
progressive chain and the result's fields."""
import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.distill import DistillConfig, Distiller, ProgressiveDistiller, compute_accuracy, softmax_temp


def _numel(model):
    return sum(p.numel() for p in model.parameters())


def _onehot(n, classes):
    return torch.nn.functional.one_hot(torch.arange(n) % classes, classes).float()


def _teacher(i, h, o):
    return nn.Sequential().add(nn.Linear(i, h)).add(nn.ReLU()).add(nn.Linear(h, o))


def test_generated_student_is_smaller():
    teacher = (nn.Sequential().add(nn.Linear(32, 128)).add(nn.ReLU()).add(nn.Linear(128, 128)).add(nn.ReLU())
               .add(nn.Linear(128, 64)).add(nn.ReLU()).add(nn.Linear(64, 10)))
    student = Distiller(teacher, DistillConfig()).generate_student(32, 10)
    assert _numel(student) < _numel(teacher)
    assert tuple(student(torch.randn(3, 32)).shape) == (3, 10)


def test_config_builder():
    c = DistillConfig().with_temperature(2.0).with_weights(0.5, 0.3, 0.2)
    assert (c.temperature, c.alpha, c.beta, c.gamma) == (2.0, 0.5, 0.3, 0.2)


def test_distillation_runs_and_records_its_loss():
    torch.manual_seed(0)
    d = Distiller(_teacher(8, 32, 4), DistillConfig(epochs=5, batch_size=16, lr=0.01))
    res = d.distill(torch.randn(64, 8), _onehot(64, 4), 8, 4)
    assert res.compression_ratio > 1.0
    assert len(res.loss_history) == 5 and all(l == l for l in res.loss_history)
    assert res.loss_history[-1] < res.loss_history[0]
    assert res.final_loss == res.loss_history[-1]


def test_softmax_temp_rows_sum_to_one():
    p = softmax_temp(torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]), 2.0)
    assert torch.allclose(p.sum(-1), torch.ones(2), atol=1e-5)
    assert torch.allclose(p, torch.softmax(torch.tensor([[0.5, 1.0, 1.5], [2.0, 2.5, 3.0]]), -1), atol=1e-6)


def test_accuracy_is_the_fraction_of_matching_argmax():
    model = nn.Sequential().add(nn.Linear(4, 3))
    x = torch.randn(4, 4)
    targets = _onehot(4, 3)
    acc = compute_accuracy(model, x, targets)
    assert 0.0 <= acc <= 1.0
    want = float((model(x).argmax(-1) == targets.argmax(-1)).float().mean())
    assert abs(acc - want) < 1e-6
    assert compute_accuracy(model, x, torch.nn.functional.one_hot(model(x).argmax(-1), 3).float()) == 1.0


def test_progressive_distiller_makes_one_result_per_round():
    torch.manual_seed(1)
    prog = ProgressiveDistiller(DistillConfig(epochs=3, batch_size=16, lr=0.01), 2)
    results = prog.distill(_teacher(8, 64, 4), torch.randn(32, 8), _onehot(32, 4), 8, 4)
    assert len(results) == 2
    assert _numel(results[1].student) <= _numel(results[0].student)   # each round's student is the next teacher


def test_result_metrics_are_in_range():
    torch.manual_seed(2)
    targets = torch.tensor([[1.0, 0.0, 0.0, 0.0]]).repeat(16, 1)
    res = Distiller(_teacher(8, 32, 4), DistillConfig(epochs=2, batch_size=8)).distill(torch.randn(16, 8), targets, 8, 4)
    assert 0.0 <= res.teacher_accuracy <= 1.0 and 0.0 <= res.student_accuracy <= 1.0
    assert res.compression_ratio > 0.0
