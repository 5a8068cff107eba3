"""gui.py, interactive.py, fused.py, quant.py: one test per behaviour of rust-nn src/gui.rs:330-380,
src/interactive.rs:640-690, src/fused.rs:190-270 and src/quant.rs:330-410."""
import math
import os
import random

import torch

from rust_neural_network_b200 import fused, gui, interactive, nn, quant


# ------------------------------------------------------------------ gui
def test_model_dashboard_html():
    h = gui.ModelDashboard.new("MLP").layer("Linear", 10, 20, "he").layer("ReLU", 20, 20, "").layer("Linear", 20, 5, "he").render()
    assert "<html" in h and "Linear" in h and "Parameters" in h


def test_training_dashboard_html():
    d = gui.TrainingDashboard.new("Run")
    d.add_point(1, 3.0)
    d.add_point(2, 1.0)
    h = d.render()
    assert "<svg" in h and "polyline" in h


def test_training_dashboard_without_points():
    assert "No data" in gui.TrainingDashboard.new("E").render()


def test_tensor_heatmap():
    h = gui.tensor_heatmap_html(torch.tensor([[1.0, 2.0], [3.0, 4.0]]), 100)
    assert h.count("<td") == 4 and "hsl(" in h


def test_full_dashboard_has_both_sections():
    t = gui.TrainingDashboard.new("T")
    t.add_point(1, 1.0)
    h = gui.full_dashboard("Full", gui.ModelDashboard.new("M").layer("Linear", 4, 8, "he"), t)
    assert "Architecture" in h and "Metrics" in h


def test_launch_writes_the_file(tmp_path):
    path = str(tmp_path / "gui.html")
    gui.launch("<html>test</html>", path)
    assert os.path.exists(path) and open(path).read() == "<html>test</html>"


# ------------------------------------------------------------------ interactive
def test_sparkline_rendering():
    s = interactive.sparkline([10.0, 8.0, 5.0, 3.0, 1.0])
    assert len(s) == 5 and s[0] == "█" and s[-1] == "▁"


def test_sparkline_of_a_constant():
    assert set(interactive.sparkline([5.0, 5.0, 5.0])) == {"█"}


def test_command_model_build():
    s = interactive.Session.new()
    assert "New model" in interactive.process_command(s, "model new")
    assert "Linear(4 -> 2)" in interactive.process_command(s, "model add linear 4 2")
    assert s.model is not None and s.model_input_dim == 4 and s.model_output_dim == 2


def test_command_synthetic_data():
    s = interactive.Session.new()
    assert "synthetic" in interactive.process_command(s, "data synthetic 50 3 2")
    assert s.dataset is not None and len(s.feature_columns) == 3 and s.target_column == "label"


def test_command_info():
    s = interactive.Session.new()
    s.model = nn.Sequential()
    assert "model: true" in interactive.process_command(s, "info")


# ------------------------------------------------------------------ fused
def test_fused_linear_relu_is_not_negative():
    x = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    w = torch.tensor([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]])
    b = torch.tensor([0.1, 0.2])
    y = fused.fused_linear(x, w, b, fused.FusedActivation.ReLU)
    none = fused.fused_linear(x, w, b, fused.FusedActivation.None_)
    assert y.numel() == 4 and bool((y >= 0).all())
    assert torch.allclose(none, torch.tensor([[1.1, 2.2], [4.1, 5.2]]), atol=1e-5)


def test_fused_linear_without_bias():
    y = fused.fused_linear(torch.tensor([[1.0, 2.0], [3.0, 4.0]]), torch.eye(2), None, fused.FusedActivation.None_)
    assert y.reshape(-1).tolist() == [1.0, 2.0, 3.0, 4.0]


def test_fused_linear_gelu_values():
    y = fused.fused_linear(torch.tensor([[0.0, 1.0], [-1.0, 2.0]]), torch.eye(2), None, fused.FusedActivation.GELU).reshape(-1).tolist()
    assert abs(y[0]) < 0.01 and 0.8 < y[1] < 0.85 and -0.17 < y[2] < -0.15 and 1.94 < y[3] < 1.96


def test_sparse_topk_routes_to_the_largest_logits():
    logits = torch.tensor([1.0, 3.0, 2.0, 0.0, 0.0, 0.5, 4.0, 1.0])
    idx, w = fused.sparse_topk_route(logits, 2, 4, 2)
    assert idx.tolist() == [1, 2, 2, 3]
    assert abs(float(w[0] + w[1]) - 1.0) < 1e-5 and abs(float(w[0]) - 1 / (1 + math.exp(-1.0))) < 1e-5


def test_sparse_topk_with_k_equal_to_the_expert_count():
    idx, w = fused.sparse_topk_route(torch.tensor([1.0, 2.0, 3.0]), 1, 3, 3)
    assert idx.tolist() == [2, 1, 0] and abs(float(w.sum()) - 1.0) < 1e-5


# ------------------------------------------------------------------ quant (rotors)
def test_rotor_rotation_is_orthogonal():
    rng = random.Random(42)
    for _ in range(100):
        r = torch.tensor(quant.Rotor.random(rng).rotation_matrix())
        assert torch.allclose(r @ r.t(), torch.eye(3), atol=1e-4)


def test_sandwich_inverse_round_trips():
    r = quant.Rotor.random(random.Random(7))
    x = [0.0, 0.3, -1.7, 2.1, 0.0, 0.0, 0.0, 0.0]
    back = r.inv_sandwich(r.sandwich(x))
    assert max(abs(a - b) for a, b in zip(x, back)) < 1e-5


def test_rotorquant_error_is_a_small_fraction_of_the_range():
    dim = 12
    data = torch.tensor([i * 0.37 - 1.5 for i in range(dim)])
    q = quant.RotorQuant.with_seed(dim, 4, 123).quantize(data)
    assert float((q - data).abs().max()) < 0.15 * float(data.max() - data.min())


def test_rotorquant_keeps_shape_when_dim_is_not_a_multiple_of_three():
    t = torch.arange(20.0).reshape(2, 10)
    assert list(quant.RotorQuant.new(10, 3).quantize(t).shape) == [2, 10]


def test_rotorquant_batched_2d():
    assert list(quant.RotorQuant.new(6, 4).quantize(torch.randn(5, 6)).shape) == [5, 6]
