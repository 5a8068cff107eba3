"""error.py, one test per behaviour of rust-nn src/error.rs:244-270 plus the variants' messages (src/error.rs:70-117)."""
import pytest

from rust_neural_network_b200 import error as E
from rust_neural_network_b200.tensor import Tensor


def test_shape_mismatch_display():
    e = E.RustNnError.shape_mismatch("matmul", [2, 3], [4, 5], "A's columns must equal B's rows")
    assert isinstance(e, E.ShapeMismatch)
    assert str(e) == "matmul: shape mismatch - expected [2, 3], got [4, 5]. A's columns must equal B's rows"


def test_invalid_ndims_display():
    e = E.RustNnError.invalid_ndims("layer_norm", 2, 1)
    assert isinstance(e, E.InvalidNdims) and "expected 2 dimensions" in str(e) and str(e).startswith("layer_norm:")


def test_every_variant_is_an_exception_with_the_reference_message():
    assert "empty" in str(E.EmptyTensor("test")) and isinstance(E.EmptyTensor("test"), Exception)
    assert str(E.InvalidInput("adam", "negative learning rate")) == "adam: invalid input - negative learning rate"
    assert str(E.IndexOutOfBounds("get", [3, 0], [2, 2])) == "get: index [3, 0] is out of bounds for shape [2, 2]"
    assert str(E.Serialization("bad magic")) == "serialization error: bad magic"
    assert str(E.DeviceError("no device")) == "device error: no device"
    assert str(E.DataLoad("missing file")) == "data loading error: missing file"
    for cls in (E.ShapeMismatch, E.InvalidNdims, E.InvalidInput, E.IndexOutOfBounds, E.EmptyTensor, E.Serialization, E.DeviceError, E.DataLoad):
        assert issubclass(cls, E.RustNnError)


def test_from_io_wraps_the_message():
    e = E.from_io("load_csv", OSError(2, "No such file"))
    assert isinstance(e, E.InvalidInput) and str(e).startswith("load_csv: invalid input - ") and "No such file" in str(e)


def test_checked_operations_raise_the_matching_variant():
    a, b = Tensor.zeros([2, 3]), Tensor.zeros([4, 5])
    with pytest.raises(E.ShapeMismatch, match="matmul: shape mismatch"):
        E.checked_matmul(a, b)
    with pytest.raises(E.InvalidNdims, match="expected 2 dimensions, got 1"):
        E.checked_matmul(Tensor.zeros([3]), b)
    with pytest.raises(E.ShapeMismatch, match="reshape"):
        E.checked_reshape(a, [4, 2])
    with pytest.raises(E.ShapeMismatch, match="add"):
        E.checked_add(a, b)
    with pytest.raises(E.InvalidNdims, match="weights: expected 2 dimensions, got 1"):
        E.validate_ndims(Tensor.zeros([4]), "weights", 2)              # the reference's argument order
    with pytest.raises(E.EmptyTensor, match="softmax: input tensor is empty"):
        E.validate_non_empty(Tensor.zeros([0, 3]), "softmax")
    assert E.checked_matmul(a, Tensor.zeros([3, 4])).shape() == [2, 4]
