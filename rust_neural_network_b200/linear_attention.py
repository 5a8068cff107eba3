"""Linear (kernelised) attention (rust-nn src/linear_attention.rs): `KernelKind`, `LinearAttention`,
`linear_attention_forward`, `linear_attention_backward`. The chunked GEMM formulation lives in
`ops.linear_attention`; this module is the reference's public surface."""
import enum

from .ops.linear_attention import (LinearAttention, LinearAttentionLayer, linear_attention, linear_attention_backward,  # noqa: F401
                                   linear_attention_forward, linear_attention_ref, phi)


class KernelKind(enum.IntEnum):
    """`Elu`: phi(x) = elu(x) + 1; `Relu2`: phi(x) = max(0, x)^2."""
    Elu = 0
    Relu2 = 1

    def to_u8(self) -> int:
        return int(self)

    @staticmethod
    def from_u8(v: int) -> "KernelKind":
        return KernelKind.Relu2 if v == 1 else KernelKind.Elu


from ._compat import install as _install  # noqa: E402

_install(globals(), imported=True)
