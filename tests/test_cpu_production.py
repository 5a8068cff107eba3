"""Robustness suite (the reference's tests/production.rs, 27 cases): checked ops reject bad shapes with typed errors,
degenerate tensors (zero-sized, 0-d, single element) behave, numerically extreme inputs stay finite, serialization rejects
malformed input, results are deterministic and tensors can cross threads."""
import math
import threading

import pytest
import torch

from rust_neural_network_b200 import activations as A
from rust_neural_network_b200 import error as E
from rust_neural_network_b200 import serialize as S
from rust_neural_network_b200.tensor import Tensor


def T(data, shape):
    return Tensor.from_vec(data, shape)


def test_checked_matmul_rejects_shape_mismatch():
    with pytest.raises(E.ShapeMismatch):
        E.checked_matmul(T([0.0] * 6, [2, 3]), T([0.0] * 8, [4, 2]))


def test_checked_matmul_succeeds_on_valid_input():
    out = E.checked_matmul(T([1, 2, 3, 4, 5, 6], [2, 3]), T([1, 0, 0, 1, 1, 1], [3, 2]))
    assert out.shape() == [2, 2] and out.data().tolist() == [[4.0, 5.0], [10.0, 11.0]]


def test_checked_matmul_rejects_non_2d():
    with pytest.raises(E.DimensionError):
        E.checked_matmul(T([0.0] * 8, [2, 2, 2]), T([0.0] * 4, [2, 2]))


def test_checked_reshape_rejects_count_mismatch():
    with pytest.raises(E.ShapeMismatch):
        E.checked_reshape(T([0.0] * 6, [2, 3]), [4, 2])


def test_checked_reshape_succeeds_on_valid():
    assert E.checked_reshape(T([0.0] * 6, [2, 3]), [3, 2]).shape() == [3, 2]


def test_checked_add_rejects_incompatible():
    with pytest.raises(E.ShapeMismatch):
        E.checked_add(T([0.0] * 6, [2, 3]), T([0.0] * 4, [2, 2]))


def test_checked_add_allows_broadcast():
    out = E.checked_add(T([1.0] * 6, [2, 3]), T([1, 2, 3], [3]))
    assert out.data().tolist() == [[2.0, 3.0, 4.0], [2.0, 3.0, 4.0]]


def test_validate_ndims_works():
    E.validate_ndims(T([0.0] * 4, [2, 2]), 2)
    with pytest.raises(E.DimensionError):
        E.validate_ndims(T([0.0] * 4, [4]), 2, "weights")


def test_validate_non_empty_works():
    E.validate_non_empty(T([1.0], [1]))
    with pytest.raises(E.EmptyTensor):
        E.validate_non_empty(Tensor.zeros([0, 3]))


def test_errors_share_a_base_class_and_carry_context():
    for cls in (E.ShapeMismatch, E.DimensionError, E.InvalidArgument, E.EmptyTensor, E.SerializationError, E.IoError, E.DeviceError, E.NumericalError):
        assert issubclass(cls, E.RustNnError)
    err = E.from_io(OSError(2, "No such file"))
    assert isinstance(err, E.IoError) and "No such file" in str(err)


def test_tensor_zero_dimension():
    t = Tensor.zeros([0, 5])
    assert t.is_empty() and t.len() == 0 and t.shape() == [0, 5]
    assert t.add(t).shape() == [0, 5] and float(t.sum().data()) == 0.0


def test_tensor_scalar():
    t = Tensor(torch.tensor(3.5))
    assert t.ndim() == 0 and t.len() == 1 and t.mean() == 3.5
    assert float(t.mul(t).data()) == pytest.approx(12.25)


def test_tensor_single_element():
    t = T([-2.0], [1, 1])
    assert t.relu().get([0, 0]) == 0.0 and t.argmax() == 0 and t.max() == t.min() == -2.0


def test_matmul_1x1():
    assert T([3.0], [1, 1]).matmul(T([4.0], [1, 1])).get([0, 0]) == 12.0


def test_matmul_large_narrow():
    a, b = Tensor.ones([1, 2048]), Tensor.ones([2048, 1])
    assert a.matmul(b).get([0, 0]) == 2048.0
    assert b.matmul(a).shape() == [2048, 2048]


def test_reshape_roundtrip():
    t = T(list(range(24)), [2, 3, 4])
    assert torch.equal(t.reshape([6, 4]).reshape([2, 3, 4]).data(), t.data())
    assert t.transpose().shape() == [4, 3, 2]                     # reverses ALL axes, like the reference


def test_relu_negative_input():
    assert T([-1e30, -1.0, -0.0, 0.0], [4]).relu().data().tolist() == [0.0, 0.0, 0.0, 0.0]


def test_sigmoid_extreme_values():
    out = T([-1e4, -100.0, 0.0, 100.0, 1e4], [5]).sigmoid().data()
    assert torch.isfinite(out).all() and out[0] == 0.0 and out[2] == 0.5 and out[4] == 1.0


def test_clamp_out_of_range():
    assert T([-5.0, 0.5, 5.0], [3]).clamp(-1.0, 1.0).data().tolist() == [-1.0, 0.5, 1.0]
    assert T([0.4, 0.6, -1.5], [3]).round().data().tolist() == [0.0, 1.0, -2.0]


def test_display_formats_tensor():
    s = repr(T([1.0, 2.0], [2]))
    assert "1." in s and "2." in s


def test_softmax_sums_to_one():
    out = A.softmax(torch.tensor([[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]]))
    assert torch.allclose(out.sum(-1), torch.ones(2)) and out[1].tolist() == pytest.approx([1 / 3] * 3)


def test_softmax_extreme_values_stable():
    out = A.softmax(torch.tensor([[1e4, 1e4 - 1.0, -1e4], [-1e30, 0.0, 1e30]]))
    assert torch.isfinite(out).all() and torch.allclose(out.sum(-1), torch.ones(2))
    assert out[1, 2] == 1.0


def test_layer_norm_stable_with_extreme_input():
    x = Tensor(torch.tensor([[1e6, 1e6 + 1, 1e6 + 2, 1e6 + 3], [1e-6, 2e-6, 3e-6, 4e-6], [5.0, 5.0, 5.0, 5.0]]))
    out = x.layer_norm(Tensor.ones([4]), Tensor.zeros([4])).data()
    assert torch.isfinite(out).all() and out[2].abs().max() < 1e-2        # a constant row normalises to ~0, not NaN


def test_cross_entropy_stable_with_large_logits():
    logits = Tensor(torch.tensor([[1e4, 0.0, -1e4], [-1e4, 1e4, 0.0]]), requires_grad=True)
    target = Tensor(torch.tensor([[1.0, 0.0, 0.0], [0.0, 0.0, 1.0]]))
    loss = logits.cross_entropy_logits(target)
    loss.backward()
    assert math.isfinite(float(loss.data())) and torch.isfinite(logits.grad()).all()
    # row 0 is right (0); row 1's probability underflows and is clamped at 1e-12 like the reference (src/tensor.rs:464-496)
    assert float(loss.data()) == pytest.approx(-math.log(1e-12) / 2, rel=1e-4)


def test_serialization_rejects_invalid_magic():
    with pytest.raises(E.SerializationError):
        S.deserialize(b"XXXX" + b"\x00" * 16)
    with pytest.raises(E.SerializationError):
        S.deserialize(b"RN")                                       # truncated header


def test_serialization_rejects_truncated_payload_and_bad_version():
    blob = S.serialize([("w", torch.arange(6.0).reshape(2, 3))])
    with pytest.raises(E.SerializationError):
        S.deserialize(blob[:-4])
    with pytest.raises(E.SerializationError):
        S.deserialize(blob[:4] + (99).to_bytes(4, "little") + blob[8:])


def test_serialization_empty_dataset():
    blob = S.serialize([])
    assert S.deserialize(blob) == [] and blob[:4] == b"RNNB"


def test_matmul_is_deterministic():
    torch.manual_seed(0)
    a, b = Tensor.randn([37, 53]), Tensor.randn([53, 29])
    assert torch.equal(a.matmul(b).data(), a.matmul(b).data())


def test_tensor_send_sync():
    """A tensor built on one thread is usable from another (the reference pins `Tensor: Send + Sync`)."""
    t = Tensor.ones([4, 4])
    out = {}

    def work():
        out["v"] = float(t.matmul(t).sum().data())

    th = threading.Thread(target=work)
    th.start(); th.join()
    assert out["v"] == 64.0
