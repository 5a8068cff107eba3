"""Checkpoints: the byte-exact `rnnb` v1 container of rust-nn (src/serialize.rs) and F32 safetensors.

`serialize` / `deserialize` work on `(name, tensor)` lists; `save_model` names parameters `param_{i}`
in `parameters()` order (src/serialize.rs:96-104) and `load_model` assigns in place after a count
check (src/serialize.rs:125-140). The encoding, decoding and file I/O (atomic write, mmap read)
are done by the C++ host library; tensors are always stored as fp32 (bf16 models save their fp32
master weights). Optimizer state, step counter and RNG go to a sidecar file under reserved names
(`__opt__.*`) so the main file stays loadable by the reference.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from . import _native as nv
from .error import SerializationError

_SIGS = {
    "b200_rnnb_size": [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_longlong)],
    "b200_rnnb_serialize": [C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_longlong),
                            C.POINTER(C.c_longlong), C.POINTER(C.c_void_p), C.c_void_p, C.c_longlong],
    "b200_rnnb_header": [C.c_void_p, C.c_longlong, C.POINTER(C.c_int)],
    "b200_rnnb_index": [C.c_void_p, C.c_longlong, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_int), C.POINTER(C.c_int),
                        C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)],
    "b200_file_write_atomic": [C.c_char_p, C.c_void_p, C.c_longlong],
    "b200_file_size": [C.c_char_p],
    "b200_file_read": [C.c_char_p, C.c_void_p, C.c_longlong],
    "b200_safetensors_size": [C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)],
    "b200_safetensors_export": [C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_longlong),
                                C.POINTER(C.c_longlong), C.POINTER(C.c_void_p), C.c_void_p, C.c_longlong],
    "b200_safetensors_index": [C.c_void_p, C.c_longlong, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_int), C.POINTER(C.c_int),
                               C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)],
}
nv.register_sigs(_SIGS)

_ERR = {1: "bad magic (not an rnnb file)", 2: "unsupported rnnb version", 3: "truncated data", 4: "tensor too large for rnnb (numel is a u32)",
        5: "bad argument", 6: "system I/O error", 7: "malformed safetensors header", 8: "shape / numel mismatch"}


def _lib():
    lib = nv.host()
    lib.b200_rnnb_size.restype = C.c_longlong
    lib.b200_safetensors_size.restype = C.c_longlong
    lib.b200_file_size.restype = C.c_longlong
    lib.b200_file_read.restype = C.c_longlong
    return lib


def _check(rc: int):
    if rc != 0:
        raise SerializationError(_ERR.get(rc, f"error {rc}"))


def _pack_args(named: Sequence[Tuple[str, torch.Tensor]]):
    n = len(named)
    names_b = [nm.encode("utf-8") for nm, _ in named]
    arrs = [t.detach().to(torch.float32).cpu().contiguous().numpy() for _, t in named]
    names = (C.c_char_p * n)(*names_b)
    name_lens = (C.c_int * n)(*[len(b) for b in names_b])
    ndims = (C.c_int * n)(*[a.ndim for a in arrs])
    dims = [d for a in arrs for d in a.shape]
    dims_flat = (C.c_longlong * max(1, len(dims)))(*dims)
    numels = (C.c_longlong * n)(*[a.size for a in arrs])
    data = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
    return n, names, name_lens, ndims, dims_flat, numels, data, arrs


def serialize(named: Sequence[Tuple[str, torch.Tensor]]) -> bytes:
    """Encode `(name, tensor)` pairs as an rnnb v1 byte string."""
    lib = _lib()
    n, names, name_lens, ndims, dims_flat, numels, data, keep = _pack_args(named)
    size = lib.b200_rnnb_size(n, name_lens, ndims, numels)
    if size < 0:
        raise SerializationError(_ERR[4])
    out = np.empty(size, dtype=np.uint8)
    _check(lib.b200_rnnb_serialize(n, names, name_lens, ndims, dims_flat, numels, data, out.ctypes.data, size))
    return out.tobytes()


def deserialize(buf: bytes, requires_grad: bool = True) -> List[Tuple[str, torch.Tensor]]:
    """Decode an rnnb v1 byte string into `(name, tensor)` pairs (fp32, `requires_grad=True` as the
    reference does, src/serialize.rs:55-93)."""
    lib = _lib()
    arr = np.frombuffer(buf, dtype=np.uint8)
    cnt = C.c_int(0)
    _check(lib.b200_rnnb_header(arr.ctypes.data, arr.size, C.byref(cnt)))
    n = cnt.value
    name_off = (C.c_longlong * max(1, n))(); name_len = (C.c_int * max(1, n))(); ndim = (C.c_int * max(1, n))()
    dims_off = (C.c_longlong * max(1, n))(); numel = (C.c_longlong * max(1, n))(); data_off = (C.c_longlong * max(1, n))()
    _check(lib.b200_rnnb_index(arr.ctypes.data, arr.size, n, name_off, name_len, ndim, dims_off, numel, data_off))
    out = []
    for i in range(n):
        name = bytes(arr[name_off[i]:name_off[i] + name_len[i]]).decode("utf-8")
        shape = np.frombuffer(buf, dtype="<u8", count=ndim[i], offset=dims_off[i]).astype(np.int64).tolist() if ndim[i] else []
        data = np.frombuffer(buf, dtype="<f4", count=numel[i], offset=data_off[i]).copy()
        t = torch.from_numpy(data).view(*shape) if shape else torch.from_numpy(data).view(())
        t.requires_grad_(requires_grad)
        out.append((name, t))
    return out


def save_model(model) -> bytes:
    """rnnb bytes of `model.parameters()` named param_0, param_1, ... (file I/O is the caller's, as in the reference)."""
    return serialize([(f"param_{i}", p) for i, p in enumerate(model.parameters())])


def save_model_named(model, names: Sequence[str] | None = None) -> bytes:
    """`save_model` with the caller's names: `names[i]` for parameter i, `param_i` where the list is short
    (src/serialize.rs:107-122). A list of (name, tensor) pairs in place of the model is written as it is."""
    if names is None and not hasattr(model, "parameters"):
        return serialize(model)
    names = list(names or [])
    return serialize([(names[i] if i < len(names) else f"param_{i}", p) for i, p in enumerate(model.parameters())])


def load_model(model, buf: bytes) -> int:
    """Assign checkpoint tensors to the model's parameters in order; count and shapes must match. Returns how many
    tensors were loaded (src/serialize.rs:125-141)."""
    loaded = deserialize(buf, requires_grad=False)
    params = model.parameters()
    if len(loaded) != len(params):
        raise SerializationError(f"parameter count mismatch: checkpoint has {len(loaded)}, model has {len(params)}")
    with torch.no_grad():
        for (name, t), p in zip(loaded, params):
            if tuple(t.shape) != tuple(p.shape):
                raise SerializationError(f"shape mismatch for {name}: {tuple(t.shape)} vs {tuple(p.shape)}")
            p.copy_(t.to(p.device))
    return len(loaded)


def write_file(path: str, buf: bytes) -> None:
    """Atomic write (temp file + rename)."""
    arr = np.frombuffer(buf, dtype=np.uint8)
    _check(_lib().b200_file_write_atomic(str(path).encode(), arr.ctypes.data, arr.size))


def read_file(path: str) -> bytes:
    lib = _lib()
    size = lib.b200_file_size(str(path).encode())
    if size < 0:
        raise SerializationError(f"cannot stat {path}")
    out = np.empty(max(size, 1), dtype=np.uint8)
    got = lib.b200_file_read(str(path).encode(), out.ctypes.data, size)
    if got != size:
        raise SerializationError(f"short read from {path}")
    return out[:size].tobytes()


def save_checkpoint(path: str, model, optimizer=None, extra: Dict[str, torch.Tensor] | None = None, write_rank: int | None = 0) -> None:
    """Weights to `path` (reference-loadable); optimizer state / step / extras to `path + '.opt'`.
    With a sharded data-parallel optimizer this is a collective: every rank calls it (`prepare_checkpoint`
    all-gathers the master weights and moments) and only `write_rank` (default: rank 0) writes the files;
    `write_rank=None` lets every rank write (tensor-parallel models: each rank saves its own shards to its own path)."""
    if optimizer is not None and hasattr(optimizer, "prepare_checkpoint"):
        optimizer.prepare_checkpoint()
        import torch.distributed as dist
        if write_rank is not None and dist.is_initialized() and dist.get_rank(getattr(optimizer, "group", None)) != write_rank:
            return
    write_file(path, save_model(model))
    if optimizer is not None or extra:
        side = []
        if optimizer is not None:
            side += _optimizer_named(model, optimizer)
        for k, v in (extra or {}).items():
            side.append((f"__extra__.{k}", v))
        write_file(str(path) + ".opt", serialize(side))


def _optimizer_named(model, optimizer):
    """Optimizer state as named tensors. State vectors that span the optimizer's flat parameter space are cut into one
    tensor per model parameter (`__opt__.m.param_3`, in `model.parameters()` order), so a file does not depend on how an
    optimizer lays its buffers out (a sharded data-parallel optimizer orders them differently from a local one)."""
    out = []
    subs = getattr(optimizer, "opts", None)
    for j, opt in enumerate(subs if subs is not None else [optimizer]):
        flat = getattr(opt, "flat", None)
        tag = f"@{j}" if subs is not None else ""
        for k, v in opt.state_tensors().items():
            if flat is not None and v.dim() == 1 and v.numel() == flat.numel:
                for i, p in enumerate(model.parameters()):
                    o = flat.offsets.get(id(p))
                    if o is not None:
                        out.append((f"__opt__.{k}.param_{i}", v[o:o + p.numel()].view(p.shape)))
            else:
                out.append((f"__opt__.{k}{tag}", v))
    return out


def load_checkpoint(path: str, model, optimizer=None) -> Dict[str, torch.Tensor]:
    load_model(model, read_file(path))
    extra = {}
    import os
    if os.path.exists(str(path) + ".opt"):
        subs = getattr(optimizer, "opts", None) or ([optimizer] if optimizer is not None else [])
        state = optimizer.state_tensors() if optimizer is not None else {}
        params = list(model.parameters())
        for name, t in deserialize(read_file(str(path) + ".opt"), requires_grad=False):
            if name.startswith("__opt__.") and optimizer is not None:
                key = name[len("__opt__."):]
                dst = None
                if ".param_" in key:
                    k, idx = key.rsplit(".param_", 1)
                    p = params[int(idx)] if int(idx) < len(params) else None
                    for opt in subs:                      # the optimizer that owns this parameter
                        flat = getattr(opt, "flat", None)
                        o = flat.offsets.get(id(p)) if (flat is not None and p is not None) else None
                        if o is not None and k in opt.state_tensors():
                            dst = opt.state_tensors()[k][o:o + p.numel()]
                else:
                    dst = state.get(key)
                if dst is not None:
                    with torch.no_grad():
                        dst.copy_(t.to(dst.device).reshape(dst.shape))
            elif name.startswith("__extra__."):
                extra[name[len("__extra__."):]] = t
    for opt in (getattr(optimizer, "opts", None) or ([optimizer] if optimizer is not None else [])):
        if getattr(opt, "flat", None) is not None and opt.flat.shadow is not None:
            with torch.no_grad():
                opt.flat.shadow.copy_(opt.flat.master)
    return extra


def safetensors_export(named: Sequence[Tuple[str, torch.Tensor]]) -> bytes:
    lib = _lib()
    n, names, name_lens, ndims, dims_flat, numels, data, keep = _pack_args(named)
    size = lib.b200_safetensors_size(n, names, name_lens, ndims, dims_flat, numels)
    out = np.empty(size, dtype=np.uint8)
    _check(lib.b200_safetensors_export(n, names, name_lens, ndims, dims_flat, numels, data, out.ctypes.data, size))
    return out.tobytes()


def safetensors_import(buf: bytes) -> List[Tuple[str, torch.Tensor]]:
    """F32 tensors of a safetensors blob in file order (`__metadata__` is skipped; the reference's
    importer neither skips it nor keeps the order, src/serialize.rs:212-247)."""
    lib = _lib()
    arr = np.frombuffer(buf, dtype=np.uint8)
    cap = 4096
    while True:
        name_off = (C.c_longlong * cap)(); name_len = (C.c_int * cap)(); ndim = (C.c_int * cap)()
        dims = (C.c_longlong * (cap * 8))(); db = (C.c_longlong * cap)(); de = (C.c_longlong * cap)()
        base = C.c_longlong(0)
        n = lib.b200_safetensors_index(arr.ctypes.data, arr.size, cap, name_off, name_len, ndim, dims, db, de, C.byref(base))
        if n < 0:
            raise SerializationError(_ERR.get(-n, f"error {-n}"))
        if n <= cap:
            break
        cap = n
    out = []
    for i in range(n):
        name = bytes(arr[name_off[i]:name_off[i] + name_len[i]]).decode("utf-8")
        shape = [dims[i * 8 + k] for k in range(ndim[i])]
        cnt = (de[i] - db[i]) // 4
        data = np.frombuffer(buf, dtype="<f4", count=cnt, offset=base.value + db[i]).copy()
        out.append((name, torch.from_numpy(data).view(*shape) if shape else torch.from_numpy(data).view(())))
    return out


# The reference exports both a module and a function called `serialize` from its crate root; the module
# object is made callable so that `pkg.serialize(named)` and `pkg.serialize.load_model` both work.
import sys as _sys
import types as _types


class _CallableModule(_types.ModuleType):
    def __call__(self, *args, **kwargs):
        return serialize(*args, **kwargs)


_sys.modules[__name__].__class__ = _CallableModule


from ._compat import install as _install  # noqa: E402

_install(globals())
