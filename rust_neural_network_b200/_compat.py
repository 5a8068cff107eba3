"""The reference-shaped `Tensor` wrapper as an argument everywhere.

rust-nn's public functions and methods take `&Tensor` (src/activations.rs:6, src/loss.rs, src/quantize.rs:85, ...). Here
the kernels work on `torch.Tensor`; `tensor.Tensor` is the thin wrapper with the reference's method names. `install`
makes every public function of a module, and every public method of the classes it defines, accept the wrapper wherever
it accepts a `torch.Tensor`: wrapped arguments (also inside lists, tuples and (name, tensor) pairs) are unwrapped, and
if any argument was wrapped, tensors in the result come back wrapped. A call without wrappers takes one `isinstance`
scan over its arguments and is otherwise untouched.
"""
from __future__ import annotations

import functools
import inspect

import torch

from .tensor import Tensor as _W


class NewMixin:
    """`Type.new(...)`: the reference's spelling of a constructor call (`Linear::new(2, 8, true)`)."""

    @classmethod
    def new(cls, *args, **kwargs):
        return cls(*args, **kwargs)


class _Alias:
    """Read access to a field under the reference's name. A non-data descriptor: an instance attribute of the same name
    (set by the class or by the user) takes precedence, so adding an alias can never break an assignment."""

    def __init__(self, fn):
        self.fn = fn

    def __get__(self, obj, owner=None):
        return self if obj is None else self.fn(obj)


def alias_fields(cls, **fields) -> None:
    """`alias_fields(LayerNorm, num_features="n")`: `ln.num_features` reads `ln.n`; a callable computes the value."""
    for ref_name, ours in fields.items():
        setattr(cls, ref_name, _Alias((lambda self, _o=ours: getattr(self, _o)) if isinstance(ours, str) else ours))


def _has_wrapped(args, kwargs) -> bool:
    for v in args:
        if isinstance(v, _W):
            return True
        if isinstance(v, (list, tuple)):
            for u in v:
                if isinstance(u, _W) or (isinstance(u, tuple) and any(isinstance(w, _W) for w in u)):
                    return True
    for v in kwargs.values():
        if isinstance(v, _W):
            return True
    return False


def unwrap(v):
    if isinstance(v, _W):
        return v.t
    if isinstance(v, list):
        return [unwrap(u) for u in v]
    if isinstance(v, tuple):
        return tuple(unwrap(u) for u in v)
    return v


def rewrap(v):
    if isinstance(v, torch.Tensor) and not isinstance(v, torch.nn.Parameter):
        return _W(v)
    if isinstance(v, tuple):
        return tuple(rewrap(u) for u in v)
    if isinstance(v, list):
        return [rewrap(u) for u in v]
    return v


def accept_wrapped(fn):
    if getattr(fn, "_accepts_wrapped", False):
        return fn

    @functools.wraps(fn)
    def inner(*args, **kwargs):
        if not _has_wrapped(args, kwargs):
            return fn(*args, **kwargs)
        return rewrap(fn(*[unwrap(a) for a in args], **{k: unwrap(v) for k, v in kwargs.items()}))

    inner._accepts_wrapped = True
    return inner


def _wrap_class(cls) -> None:
    if not hasattr(cls, "new"):                      # `Type.new(...)` for classes that do not spell it out
        cls.new = classmethod(lambda c, *a, **k: c(*a, **k))
    for name, attr in list(cls.__dict__.items()):
        if name.startswith("_") and name not in ("__init__", "__call__"):
            continue
        if isinstance(attr, staticmethod):
            setattr(cls, name, staticmethod(accept_wrapped(attr.__func__)))
        elif isinstance(attr, classmethod):
            setattr(cls, name, classmethod(accept_wrapped(attr.__func__)))
        elif inspect.isfunction(attr):
            setattr(cls, name, accept_wrapped(attr))


def install(namespace: dict, skip=(), imported: bool = False) -> None:
    """Call as `install(globals())` at the end of a module. `imported`: also wrap functions that the module re-exports
    from elsewhere (only this module's binding changes)."""
    mod = namespace.get("__name__")
    for name, obj in list(namespace.items()):
        if name.startswith("_") or name in skip:
            continue
        if inspect.isfunction(obj) and (imported or obj.__module__ == mod):
            namespace[name] = accept_wrapped(obj)
        elif inspect.isclass(obj) and obj.__module__ == mod and not issubclass(obj, (BaseException, _W)) and not issubclass(obj, __import__("enum").Enum):
            _wrap_class(obj)
