"""Error types and checked operations (rust-nn src/error.rs:12-238).

`RustNnError` is the base class; its eight variants mirror the reference enum. The `checked_*`
functions validate shapes first and raise instead of panicking.
"""
from __future__ import annotations

from typing import Sequence

import torch


class RustNnError(Exception):
    """Base error (the reference's `RustNnError` enum)."""


class ShapeMismatch(RustNnError):
    def __init__(self, expected, got, context: str = ""):
        self.expected, self.got, self.context = tuple(expected), tuple(got), context
        super().__init__(f"shape mismatch{': ' + context if context else ''}: expected {self.expected}, got {self.got}")


class DimensionError(RustNnError):
    pass


class InvalidArgument(RustNnError):
    pass


class EmptyTensor(RustNnError):
    pass


class SerializationError(RustNnError):
    pass


class IoError(RustNnError):
    pass


class DeviceError(RustNnError):
    pass


class NumericalError(RustNnError):
    pass


Result = object   # the reference's `Result<T>` alias; Python raises instead


def from_io(err: OSError) -> IoError:
    return IoError(str(err))


def _t(x):
    return x.t if hasattr(x, "t") and not isinstance(x, torch.Tensor) else x


def validate_ndims(t, expected: int, context: str = "") -> None:
    nd = _t(t).dim()
    if nd != expected:
        raise DimensionError(f"{context or 'tensor'}: expected {expected} dimensions, got {nd}")


def validate_non_empty(t, context: str = "") -> None:
    if _t(t).numel() == 0:
        raise EmptyTensor(f"{context or 'tensor'} is empty")


def checked_matmul(a, b):
    ta, tb = _t(a), _t(b)
    validate_ndims(ta, 2, "matmul lhs"); validate_ndims(tb, 2, "matmul rhs")
    if ta.shape[1] != tb.shape[0]:
        raise ShapeMismatch((ta.shape[0], ta.shape[1]), tuple(tb.shape), "matmul inner dimensions")
    return a.matmul(b)


def checked_reshape(t, shape: Sequence[int]):
    n = 1
    for s in shape:
        n *= int(s)
    if n != _t(t).numel():
        raise ShapeMismatch(tuple(shape), tuple(_t(t).shape), "reshape element count")
    return t.reshape(list(shape))


def checked_add(a, b):
    ta, tb = _t(a), _t(b)
    try:
        torch.broadcast_shapes(tuple(ta.shape), tuple(tb.shape))
    except RuntimeError:
        raise ShapeMismatch(tuple(ta.shape), tuple(tb.shape), "add (not broadcastable)")
    return a.add(b) if hasattr(a, "add") else a + b
