"""Error types and checked operations (rust-nn src/error.rs:12-238).

`RustNnError` is the base class; the reference enum's eight variants are subclasses with the same names and messages. The `checked_*`
functions validate shapes first and raise instead of panicking.
"""
from __future__ import annotations

from typing import Sequence

import torch


class RustNnError(Exception):
    """Base error (the reference's `RustNnError` enum, src/error.rs:12-42). The variants are subclasses; their messages
    are the reference's `Display` strings (src/error.rs:70-117)."""

    @staticmethod
    def shape_mismatch(op: str, expected, actual, detail: str = "") -> "ShapeMismatch":
        return ShapeMismatch(expected, actual, detail, op=op)

    @staticmethod
    def invalid_ndims(op: str, expected: int, actual: int) -> "InvalidNdims":
        return InvalidNdims(op, expected, actual)


class ShapeMismatch(RustNnError):
    def __init__(self, expected, got, context: str = "", op: str = ""):
        self.expected, self.got, self.actual, self.context, self.detail, self.op = tuple(expected), tuple(got), tuple(got), context, context, op
        if op:
            msg = f"{op}: shape mismatch - expected {list(self.expected)}, got {list(self.got)}. {context}"
        else:
            msg = f"shape mismatch{': ' + context if context else ''}: expected {self.expected}, got {self.got}"
        super().__init__(msg)


class InvalidNdims(RustNnError):
    """`InvalidNdims { op, expected, actual }`; also built from one ready-made message."""

    def __init__(self, op: str, expected: int = None, actual: int = None):
        self.op, self.expected, self.actual = op, expected, actual
        super().__init__(op if expected is None else f"{op}: expected {expected} dimensions, got {actual}")


class InvalidInput(RustNnError):
    def __init__(self, op: str, msg: str = None):
        self.op, self.msg = op, msg
        super().__init__(op if msg is None else f"{op}: invalid input - {msg}")


class IndexOutOfBounds(RustNnError):
    def __init__(self, op: str, index=(), shape=()):
        self.op, self.index, self.shape = op, list(index), list(shape)
        super().__init__(f"{op}: index {self.index} is out of bounds for shape {self.shape}")


class EmptyTensor(RustNnError):
    """`EmptyTensor { op }`: "<op>: input tensor is empty"."""

    def __init__(self, op: str = "tensor"):
        self.op = op
        super().__init__(op if " " in op else f"{op}: input tensor is empty")


class Serialization(RustNnError):
    def __init__(self, msg: str = ""):
        super().__init__(msg if msg.startswith("serialization error") else f"serialization error: {msg}")


class DeviceError(RustNnError):
    def __init__(self, msg: str = ""):
        super().__init__(msg if msg.startswith("device error") else f"device error: {msg}")


class DataLoad(RustNnError):
    def __init__(self, msg: str = ""):
        super().__init__(msg if msg.startswith("data loading error") else f"data loading error: {msg}")


class IoError(DataLoad):
    """File I/O failures of the host runtime (a `DataLoad` in the reference's terms)."""


class NumericalError(RustNnError):
    """Non-finite values found by a check; no counterpart in the reference's enum."""


DimensionError = InvalidNdims          # earlier names of the same variants
InvalidArgument = InvalidInput
SerializationError = Serialization

Result = object   # the reference's `Result<T>` alias; Python raises instead


def from_io(op, err=None) -> RustNnError:
    """`from_io(op, e)` -> `InvalidInput { op, msg: e.to_string() }` (src/error.rs:125-130); with the error alone, an `IoError`."""
    if err is None:
        return IoError(str(op))
    return InvalidInput(op, str(err))


def _t(x):
    return x.t if hasattr(x, "t") and not isinstance(x, torch.Tensor) else x


def validate_ndims(t, expected, context: str = "") -> None:
    """`validate_ndims(tensor, op, expected_dims)` as in the reference (src/error.rs:224-231), or `(tensor, expected_dims[, op])`."""
    if isinstance(expected, str):
        expected, context = context, expected
    nd = _t(t).dim()
    if nd != int(expected):
        raise InvalidNdims(context or "tensor", int(expected), nd)


def validate_non_empty(t, context: str = "") -> None:
    if _t(t).numel() == 0:
        raise EmptyTensor(context or "tensor")


def checked_matmul(a, b):
    ta, tb = _t(a), _t(b)
    validate_ndims(ta, 2, "matmul lhs"); validate_ndims(tb, 2, "matmul rhs")
    if ta.shape[1] != tb.shape[0]:
        raise RustNnError.shape_mismatch("matmul", (ta.shape[0], ta.shape[1]), tuple(tb.shape), "A's columns must equal B's rows")
    return a.matmul(b)


def checked_reshape(t, shape: Sequence[int]):
    n = 1
    for s in shape:
        n *= int(s)
    if n != _t(t).numel():
        raise RustNnError.shape_mismatch("reshape", tuple(shape), tuple(_t(t).shape), "element counts differ")
    return t.reshape(list(shape))


def checked_add(a, b):
    ta, tb = _t(a), _t(b)
    try:
        torch.broadcast_shapes(tuple(ta.shape), tuple(tb.shape))
    except RuntimeError:
        raise RustNnError.shape_mismatch("add", tuple(ta.shape), tuple(tb.shape), "shapes are not broadcastable")
    return a.add(b) if hasattr(a, "add") else a + b
