"""Every public name of the reference's crate root resolves from the package root."""
import rust_neural_network_b200 as rn


def test_every_root_export_resolves():
    missing = []
    for name in rn.__all__:
        try:
            getattr(rn, name)
        except Exception as e:          # noqa: BLE001
            missing.append((name, repr(e)))
    assert not missing, missing
    assert rn.VERSION.startswith("2.1.0")
    assert rn.blas_matmul is rn.blas.matmul and rn.LinearAttentionLayer.elu(64).scale == 0.125
    assert rn.KernelKind.Relu2.to_u8() == 1 and rn.AttentionKind is rn.looped_transformer.AttentionKind
    assert rn.NativeBackend().name().startswith("native") and "tcgen05" in rn.NVIDIA_PTX_KERNEL
    assert rn.nn.NormalMoE is rn.NormalMoE


# Names of the reference with no counterpart, and why.
_NO_COUNTERPART = {
    ("type", "tensor", "TensorData"): "the reference's reference-counted storage cell; torch.Tensor is the storage here",
    ("type", "tensor", "Op"): "the reference's autograd graph nodes; torch.autograd supplies the graph",
    ("method", "QuantFormat", "name"): "an Enum member's `.name` is taken by Python; the display string is `name_str()`",
    ("method", "Value", "parse"): "a private JSON helper inside the reference's serialize module",
    ("field", "TensorData", "data"): "see TensorData", ("field", "TensorData", "grad"): "see TensorData",
    ("field", "TensorData", "requires_grad"): "see TensorData", ("field", "TensorData", "creator"): "see TensorData",
    ("field", "TensorData", "device"): "see TensorData",
}


def _public_names():
    import importlib
    import os
    import pkgutil
    classes, names = {}, set()
    for m in pkgutil.walk_packages(rn.__path__, rn.__name__ + "."):
        if any(x in m.name for x in ("._native", "._build", ".cpu_ref")):
            continue
        mod = importlib.import_module(m.name)
        for k, v in vars(mod).items():
            if k.startswith("_"):
                continue
            names.add(k)
            if isinstance(v, type) and v.__module__.startswith(rn.__name__):
                classes.setdefault(k, v)
    path = os.path.join(os.path.dirname(__file__), "reference_public_api.txt")
    rows = [tuple(l.split()) for l in open(path) if l.strip() and not l.startswith("#")]
    return classes, names, rows


def test_every_public_type_function_and_method_of_the_reference_has_a_counterpart():
    """970 names: 148 types / constants, 87 free functions (looked up in the module of the same name), the methods of
    every `impl` block and the public fields of every struct (looked up on the class of the same name)."""
    import importlib
    classes, names, rows = _public_names()
    assert len(rows) > 900
    missing = []
    for kind, where, name in rows:
        if (kind, where, name) in _NO_COUNTERPART:
            continue
        if kind == "type":
            ok = name in names or hasattr(rn, name)
        elif kind == "fn":
            ok = False
            for cand in (f"{rn.__name__}.{where}", f"{rn.__name__}.models.{where}"):
                try:
                    ok = ok or hasattr(importlib.import_module(cand), name)
                except ImportError:
                    pass
        elif kind == "method":
            cls = classes.get(where)
            ok = cls is not None and (hasattr(cls, name) or name in getattr(cls, "__annotations__", {}))
        else:                                # a public field: a class attribute / alias, a dataclass field, or set in a constructor
            cls = classes.get(where)
            ok = cls is not None and (hasattr(cls, name) or any(name in getattr(c, "__annotations__", {}) for c in cls.__mro__))
            if cls is not None and not ok:
                import inspect
                import re
                for c in cls.__mro__:
                    if c.__module__.startswith(rn.__name__) and re.search(rf"self\.{name}\b", inspect.getsource(c)):
                        ok = True
                        break
        if not ok:
            missing.append((kind, where, name))
    assert not missing, missing
