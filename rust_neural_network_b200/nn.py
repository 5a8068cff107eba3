"""Neural-network modules: the API of rust-nn's `nn.rs` on top of this package's kernels.

`Module` mirrors the reference trait (rust-nn src/nn.rs:6-12): `forward`, `parameters()` (a list,
in the order the reference enumerates them - that order is the checkpoint contract of
`save_model`, src/serialize.rs:96-104) and `set_training`. Parameters are fp32 master tensors;
when activations are bf16 the kernels read a bf16 shadow that the optimizers keep in sync.

Where the reference deviates from the intended mathematics the intended behaviour is implemented
and the difference is stated in the class docstring.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch

from .ops import functional as F
from .ops import kernels as K
from .tensor import Tensor as _Wrapped
from ._compat import NewMixin as _NewMixin

Parameter = torch.nn.Parameter


def _param(t: torch.Tensor) -> Parameter:
    return Parameter(t.float().contiguous(), requires_grad=True)


def _rewrap(out):
    if isinstance(out, torch.Tensor):
        return _Wrapped(out)
    if isinstance(out, tuple):
        return tuple(_rewrap(o) for o in out)
    return out


def _accepts_wrapped(f):
    import functools

    @functools.wraps(f)
    def forward(self, *a, **kw):
        for v in a:
            if isinstance(v, _Wrapped):
                return _rewrap(f(self, *[u.t if isinstance(u, _Wrapped) else u for u in a], **kw))
        return f(self, *a, **kw)
    return forward


class Module(_NewMixin):
    """Base class. Sub-modules and parameters are discovered through `children()` / `own_parameters()`
    overrides or, by default, by scanning instance attributes in definition order."""

    training: bool = True

    def __init_subclass__(cls, **kw):
        """Every `forward` also takes the reference-shaped `Tensor` wrapper (src/nn.rs:12 `fn forward(&self, x: &Tensor)`):
        wrapped inputs are unwrapped, and the result then comes back wrapped."""
        super().__init_subclass__(**kw)
        f = cls.__dict__.get("forward")
        if f is not None:
            cls.forward = _accepts_wrapped(f)

    def forward(self, x):
        raise NotImplementedError

    def __call__(self, *a, **kw):
        return self.forward(*a, **kw)

    # -- structure
    def children(self) -> List["Module"]:
        out = []
        for v in self.__dict__.values():
            if isinstance(v, Module):
                out.append(v)
            elif isinstance(v, (list, tuple)):
                out.extend(m for m in v if isinstance(m, Module))
        return out

    def own_parameters(self) -> List[Parameter]:
        return [v for v in self.__dict__.values() if isinstance(v, Parameter)]

    def parameters(self) -> List[Parameter]:
        """Own parameters first, then children in attribute order (override to pin another order)."""
        ps = list(self.own_parameters())
        for c in self.children():
            ps.extend(c.parameters())
        # de-duplicate shared parameters, keep first occurrence
        seen, out = set(), []
        for p in ps:
            if id(p) not in seen:
                seen.add(id(p)); out.append(p)
        return out

    def buffers(self) -> List[torch.Tensor]:
        bs = [v for k, v in self.__dict__.items() if isinstance(v, torch.Tensor) and not isinstance(v, Parameter) and k.startswith("buf_")]
        for c in self.children():
            bs.extend(c.buffers())
        return bs

    def set_training(self, training: bool) -> None:
        self.training = training
        for c in self.children():
            c.set_training(training)

    def train(self):
        self.set_training(True); return self

    def eval(self):
        self.set_training(False); return self

    def zero_grad(self):
        for p in self.parameters():
            if p.grad is not None:
                p.grad.zero_()

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    # -- placement / precision
    compute_dtype = torch.float32

    def to_device(self, device, dtype: Optional[torch.dtype] = None):
        """Move parameters and buffers; `dtype` selects the activation/compute dtype (fp32 or bf16).
        Master weights always stay fp32."""
        device = torch.device(device)
        for p in self.parameters():
            if p.device != device:
                p.data = p.data.to(device)
                if p.grad is not None:
                    p.grad = p.grad.to(device)
                if hasattr(p, "_lp"):
                    del p._lp
        self._move_buffers(device)
        if dtype is not None:
            self._set_compute_dtype(dtype)
        return self

    def _move_buffers(self, device):
        for k, v in list(self.__dict__.items()):
            if isinstance(v, torch.Tensor) and not isinstance(v, Parameter):
                self.__dict__[k] = v.to(device)
        for c in self.children():
            c._move_buffers(device)

    def _set_compute_dtype(self, dtype):
        self.compute_dtype = dtype
        for c in self.children():
            c._set_compute_dtype(dtype)

    def cuda(self, dtype=None):
        return self.to_device("cuda", dtype)

    @property
    def device(self):
        ps = self.parameters()
        return ps[0].device if ps else torch.device("cpu")


# ----------------------------------------------------------------------------- initialisers
def he_normal(shape, generator=None):
    """N(0, sqrt(2/fan_in)), fan_in = last dim (rust-nn src/tensor.rs:255-260)."""
    return torch.randn(*shape, generator=generator) * math.sqrt(2.0 / shape[-1])


def xavier_normal(shape, generator=None):
    fan_in, fan_out = shape[-1], shape[0]
    return torch.randn(*shape, generator=generator) * math.sqrt(2.0 / (fan_in + fan_out))


def kaiming_uniform(shape, generator=None):
    """U(-1/sqrt(fan_in), 1/sqrt(fan_in)) (PyTorch's nn.Linear default)."""
    bound = 1.0 / math.sqrt(shape[-1])
    return (torch.rand(*shape, generator=generator) * 2 - 1) * bound


def normal_init(std):
    return lambda shape, generator=None: torch.randn(*shape, generator=generator) * std


# ----------------------------------------------------------------------------- layers
class Linear(Module):
    """y = x W^T + b; W [out, in] He-normal, bias zeros; N-D input is flattened to 2-D
    (rust-nn src/nn.rs:20-83). `init` selects another initialiser (e.g. `kaiming_uniform`)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, init=he_normal, act: str = "none",
                 generator=None):
        self.in_features, self.out_features = in_features, out_features
        self.weight = _param(init((out_features, in_features), generator=generator))
        if bias:
            if init is kaiming_uniform:
                self.bias = _param((torch.rand(out_features, generator=generator) * 2 - 1) / math.sqrt(in_features))
            else:
                self.bias = _param(torch.zeros(out_features))
        else:
            self.bias = None
        self.act = act

    def forward(self, x, residual=None):
        return F.linear(x, self.weight, self.bias, self.act, residual)

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])


class Sequential(Module):
    """Ordered container with the reference's builder API (`Sequential::new().add(m)`, src/nn.rs:86-132).
    Linear followed by an activation module is executed as one fused GEMM epilogue."""

    def __init__(self, *layers: Module):
        self.layers: List[Module] = list(layers)

    def add(self, m: Module) -> "Sequential":
        if isinstance(m, type):              # `.add(ReLU)`: the reference's unit structs are written without parentheses
            m = m()
        self.layers.append(m)
        return self

    def children(self):
        return list(self.layers)

    def forward(self, x):
        i, n = 0, len(self.layers)
        while i < n:
            m = self.layers[i]
            nxt = self.layers[i + 1] if i + 1 < n else None
            fuse = type(m) is Linear and m.act == "none" and isinstance(nxt, _Activation) and nxt.fusable
            if fuse:
                x = F.linear(x, m.weight, m.bias, nxt.name, None)
                i += 2
            else:
                x = m(x)
                i += 1
        return x

    def parameters(self):
        ps = []
        for m in self.layers:
            ps.extend(m.parameters())
        return ps


class _Activation(Module):
    name = "none"
    fusable = True

    def forward(self, x):
        return getattr(F, self.name)(x)

    def parameters(self):
        return []


class ReLU(_Activation): name = "relu"
class Sigmoid(_Activation): name = "sigmoid"
class Tanh(_Activation): name = "tanh"
class GELU(_Activation): name = "gelu"
class SiLU(_Activation): name = "silu"


class Softmax(Module):
    """Softmax over the last axis (differentiable; the reference's is forward-only, src/activations.rs:23-62)."""

    def forward(self, x):
        return F.softmax(x)

    def parameters(self):
        return []


class Flatten(Module):
    def forward(self, x):
        return x.reshape(x.shape[0], -1)

    def parameters(self):
        return []


class Dropout(Module):
    """Inverted dropout, p clamped to [0,1] (src/nn.rs:210-259). Differentiable (the reference detaches
    its output). The mask is a stateless hash of (seed, element index); the seed advances per call."""

    def __init__(self, p: float, seed: int = 0x5EED):
        self.p = min(max(float(p), 0.0), 1.0)
        self._seed = seed
        self._calls = 0

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        self._calls += 1
        return F.dropout(x, self.p, self._seed + 7919 * self._calls)

    def parameters(self):
        return []


class LayerNorm(Module):
    """Last-axis LayerNorm, gamma=1, beta=0, eps 1e-5 (src/nn.rs:275-310)."""

    def __init__(self, n: int, eps: float = 1e-5):
        self.n, self.eps = n, eps
        self.gamma = _param(torch.ones(n))
        self.beta = _param(torch.zeros(n))

    def with_eps(self, eps: float):
        self.eps = eps
        return self

    def forward(self, x):
        return F.layer_norm(x, self.gamma, self.beta, self.eps)

    def parameters(self):
        return [self.gamma, self.beta]


class BatchNorm1D(Module):
    """BatchNorm over the batch axis of a [batch, n] input, biased variance, eps 1e-5 (src/nn.rs:327-388).
    Unlike the reference (batch statistics only, normalisation detached) this keeps running
    statistics for eval mode and back-propagates the full gradient through the normalisation."""

    def __init__(self, n: int, eps: float = 1e-5, momentum: float = 0.1):
        self.n, self.eps, self.momentum = n, eps, momentum
        self.gamma = _param(torch.ones(n))
        self.beta = _param(torch.zeros(n))
        self.buf_running_mean = torch.zeros(n)
        self.buf_running_var = torch.ones(n)

    def forward(self, x):
        if x.dim() != 2 or x.shape[1] != self.n:
            raise ValueError(f"BatchNorm1D expects [batch, {self.n}], got {tuple(x.shape)}")
        return F.batch_norm(x, self.gamma, self.beta, self.buf_running_mean, self.buf_running_var, self.eps,
                            self.momentum, self.training)

    def parameters(self):
        return [self.gamma, self.beta]


class Embedding(Module):
    """Token embedding table [vocab, dim] (the reference has none: it embeds with a Linear,
    src/looped_transformer.rs:259). N(0, std) init."""

    def __init__(self, vocab: int, dim: int, std: float = 0.02, generator=None):
        self.vocab, self.dim = vocab, dim
        self.weight = _param(torch.randn(vocab, dim, generator=generator) * std)

    def forward(self, ids):
        return F.embedding(ids, self.weight, self.compute_dtype)

    def parameters(self):
        return [self.weight]


class Recursive(Module):
    """Applies one module `depth` times (src/nn.rs:506-525)."""

    def __init__(self, module: Module, depth: int):
        self.module, self.depth = module, depth

    def forward(self, x):
        for _ in range(self.depth):
            x = self.module(x)
        return x

    def parameters(self):
        return self.module.parameters()


class RNNCell(Module):
    """h' = tanh(W_ih x + W_hh h) (src/nn.rs:535-565); `forward(x)` uses h = 0."""

    def __init__(self, input_size: int, hidden_size: int):
        self.input_size, self.hidden_size = input_size, hidden_size
        self.w_ih = Linear(input_size, hidden_size, bias=True)
        self.w_hh = Linear(hidden_size, hidden_size, bias=True)

    def step(self, x, h):
        pre = self.w_hh(h, residual=None)
        return F.tanh(F.linear(x, self.w_ih.weight, self.w_ih.bias, "none", pre))

    def forward(self, x):
        h = torch.zeros(*x.shape[:-1], self.hidden_size, dtype=x.dtype, device=x.device)
        return self.step(x, h)

    def parameters(self):
        return self.w_ih.parameters() + self.w_hh.parameters()


class FakeQuantize(Module):
    """Uniform fake quantisation: qmin=-2^(b-1), qmax=2^(b-1)-1, scale=max_val/qmax (src/nn.rs:644-667),
    with a real straight-through gradient."""

    def __init__(self, bits: int, max_val: float):
        self.bits = bits
        self.qmin, self.qmax = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
        self.scale = max_val / self.qmax

    def forward(self, x):
        return F.fake_quantize(x, self.scale, self.qmin, self.qmax)

    def parameters(self):
        return []


class _CompressedAttention(Module):
    """Shared body of CSA / HCA. The reference's versions are identity stubs that hold an unused
    compression Linear(hidden*group -> hidden) (src/nn.rs:579-629). Here `forward` is the identity
    as well (API parity) and `compress(x)` performs the group compression the Linear was sized
    for: [B, S, hidden] -> [B, S/group, hidden]."""

    def __init__(self, hidden: int, group: int):
        self.hidden, self.group = hidden, group
        self.compression = Linear(hidden * group, hidden)

    def forward(self, x):
        return x

    def compress(self, x):
        B, S, Hd = x.shape
        S2 = S // self.group
        return self.compression(x[:, : S2 * self.group].reshape(B, S2, Hd * self.group))

    def parameters(self):
        return self.compression.parameters()


class CSA(_CompressedAttention):
    pass


class HCA(_CompressedAttention):
    pass


# ----------------------------------------------------------------------------- functional attention
def attention(q, k, v, causal: bool = False):
    """softmax(q k^T / sqrt(d)) v for [B, S, d] tensors (src/nn.rs:699-706), via the flash kernel."""
    return flash_attention(q, k, v, causal)


def flash_attention(q, k, v, causal: bool = False):
    """[B, S, d] -> [B, S, d], scale 1/sqrt(d) (src/nn.rs:707-714)."""
    d = q.shape[-1]
    if q.is_cuda and d not in (64, 128):
        # other head sizes: dense path through the GEMM kernel
        # (scores on the tcgen05 GEMM, scale + causal mask + softmax in one row kernel, then the second GEMM)
        s = F.matmul(q, k.transpose(1, 2).contiguous())
        return F.matmul(F.softmax(s, 1.0 / math.sqrt(d), s.shape[-2] if causal else 0), v.contiguous())
    o = F.flash_attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), 1.0 / math.sqrt(d), causal)
    return o.squeeze(2)


def __getattr__(name):
    # NormalMoE / FineGrainedMoE live in models.moe (they pull in the routing kernels); exposed here as in src/nn.rs
    if name in ("NormalMoE", "FineGrainedMoE"):
        from .models import moe
        return getattr(moe, name)
    raise AttributeError(name)


# field names of the reference's structs (src/nn.rs:226-233, 573-576, 636-641, 690-697) beside this package's own
from ._compat import alias_fields as _alias_fields  # noqa: E402

_alias_fields(BatchNorm1D, num_features="n")
_alias_fields(LayerNorm, num_features="n")
_alias_fields(CSA, compression_layer="compression", group_size="group")
_alias_fields(HCA, compression_layer="compression", group_size="group")
_alias_fields(FakeQuantize, num_bits="bits")
_alias_fields(RNNCell, weight_ih="w_ih", weight_hh="w_hh")
