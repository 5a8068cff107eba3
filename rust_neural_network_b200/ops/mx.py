"""Block-scaled low-precision GEMM operands (csrc/gemm/gemm_mx_sm100.cu).

Two formats whose scale factors the 5th-generation tensor core applies itself (`tcgen05.mma ... .block_scale`):

* ``mxfp8``: e4m3 elements with one power-of-two (ue8m0) scale per 32 elements along K;
* ``nvfp4``: e2m1 elements, two per byte with the even element in the low nibble - the magnitude table
  {0, .5, 1, 1.5, 2, 3, 4, 6} and nibble order of the reference's NVFP4 format (src/quantize.rs:139-165) - with one
  ue4m3 scale per 16 elements and one fp32 scale per tensor (the reference stores an fp32 scale per group and
  dequantises in software; the tensor core needs the 8-bit scale).

`quantize_mx` produces an `MxTensor`, `gemm_mx(a, b)` multiplies two of them as ``a @ b.T`` with fp32 accumulation,
`dequantize_mx` restores fp32 values (the oracle of the tests and the CPU path), `MxLinear` is a Linear layer whose weight
is stored in one of the formats and whose activations are quantised on the fly.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _native as nv

KINDS = {"mxfp8": 0, "nvfp4": 1}
_VEC = {0: 32, 1: 16}
_KMULT = {0: 128, 1: 256}
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


class MxGemmArgs(C.Structure):
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("sfa", C.c_void_p), ("sfb", C.c_void_p), ("C", C.c_void_p), ("ldc", C.c_longlong),
                ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("out_f32", C.c_int), ("alpha", C.c_float), ("kind", C.c_int),
                ("status", C.c_void_p)]


nv.register_sigs({
    "b200_gemm_mx": [C.POINTER(MxGemmArgs), C.c_int, C.c_void_p],
    "b200_mx_quant": [C.c_void_p, C.c_int, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p],
    "b200_mx_dequant": [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p],
})


@dataclass
class MxTensor:
    """[rows, K] matrix in a block-scaled format. `data` holds the element bytes row by row; `sf` the scale factors in
    512-byte chunks (4 consecutive scales of 128 consecutive rows per chunk, byte (r % 32) * 16 + (r // 32) * 4 + j),
    ordered [row block of 128][chunk along K] and padded to a multiple of 256 rows."""
    data: torch.Tensor
    sf: torch.Tensor
    rows: int
    K: int
    kind: int
    tensor_scale: float = 1.0

    @property
    def nbytes(self) -> int:
        return self.data.numel() + self.sf.numel()


def _sf_bytes(rows: int, K: int, kind: int) -> int:
    return (rows + 255) // 256 * 2 * (K // (4 * _VEC[kind])) * 512


def _sf_index(rows: int, K: int, kind: int, device):
    """Byte offset of the scale factor of (row, block along K) inside the chunk buffer, as a [rows, K / V] tensor."""
    nb = K // _VEC[kind]
    r = torch.arange(rows, device=device).unsqueeze(1)
    j = torch.arange(nb, device=device).unsqueeze(0)
    rr = r % 128
    return ((r // 128) * (nb // 4) + j // 4) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + j % 4


def _e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).float()


def _quantize_torch(x: torch.Tensor, kind: int, tensor_scale: float):
    """Reference implementation in torch ops (CPU path and oracle of the kernels)."""
    rows, K = x.shape
    V = _VEC[kind]
    xb = x.float().reshape(rows, K // V, V)
    amax = xb.abs().amax(-1)
    sf = torch.zeros(_sf_bytes(rows, K, kind), dtype=torch.uint8, device=x.device)
    idx = _sf_index(rows, K, kind, x.device).reshape(-1)
    if kind == 0:
        m, ex = torch.frexp(amax / 448.0)
        e = torch.where(m > 0.5, ex, ex - 1).clamp(-127, 127)
        e = torch.where(amax > 0, e, torch.full_like(e, -127))
        sf[idx] = (e + 127).to(torch.uint8).reshape(-1)
        q = (xb * torch.ldexp(torch.ones_like(amax), -e).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
        data = q.view(torch.uint8).reshape(rows, K)
    else:
        qs = (amax / (6.0 * tensor_scale)).clamp(max=448).to(torch.float8_e4m3fn)
        sf[idx] = qs.view(torch.uint8).reshape(-1)
        s = qs.float() * tensor_scale
        inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s)).unsqueeze(-1)
        v = xb * inv
        a = v.abs()
        bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
        code = torch.bucketize(a, bounds, right=True).to(torch.uint8) | ((v < 0).to(torch.uint8) << 3)
        code = code.reshape(rows, K // 2, 2)
        data = code[..., 0] | (code[..., 1] << 4)
    return data.contiguous(), sf


def quantize_mx(x: torch.Tensor, kind: str = "mxfp8", tensor_scale: float | None = None) -> MxTensor:
    """Quantise a [rows, K] matrix (bf16 or fp32). K must be a multiple of 128 (mxfp8) or 256 (nvfp4). For nvfp4 the
    per-tensor scale defaults to absmax / (6 * 448), which puts the largest block scale at the top of ue4m3."""
    k = KINDS[kind]
    if x.dim() != 2:
        raise ValueError("quantize_mx takes a matrix")
    rows, K = x.shape
    if K % _KMULT[k] != 0:
        raise ValueError(f"K = {K} must be a multiple of {_KMULT[k]} for {kind}")
    if k == 1 and tensor_scale is None:
        tensor_scale = max(float(x.detach().abs().max()) / (6.0 * 448.0), 1e-30)
    ts = float(tensor_scale) if k == 1 else 1.0
    if not x.is_cuda:
        data, sf = _quantize_torch(x.detach(), k, ts)
        return MxTensor(data, sf, rows, K, k, ts)
    x = x.detach()
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    if x.stride(1) != 1:
        x = x.contiguous()
    data = torch.empty((rows, K if k == 0 else K // 2), dtype=torch.uint8, device=x.device)
    sf = torch.zeros(_sf_bytes(rows, K, k), dtype=torch.uint8, device=x.device)
    nv.check(nv.cuda().b200_mx_quant(x.data_ptr(), int(x.dtype == torch.bfloat16), x.stride(0), rows, K, k, ts, data.data_ptr(),
                                     sf.data_ptr(), nv.stream_ptr()), "mx_quant")
    nv.count_launch()
    return MxTensor(data, sf, rows, K, k, ts)


def dequantize_mx(t: MxTensor) -> torch.Tensor:
    """fp32 [rows, K] values the tensor core sees."""
    if t.data.is_cuda:
        out = torch.empty((t.rows, t.K), dtype=torch.float32, device=t.data.device)
        nv.check(nv.cuda().b200_mx_dequant(t.data.data_ptr(), t.sf.data_ptr(), t.rows, t.K, t.kind, t.tensor_scale, out.data_ptr(),
                                           nv.stream_ptr()), "mx_dequant")
        nv.count_launch()
        return out
    V = _VEC[t.kind]
    q = t.sf[_sf_index(t.rows, t.K, t.kind, t.data.device)]
    if t.kind == 0:
        s = torch.ldexp(torch.ones(q.shape), q.int() - 127)
        vals = _e4m3_decode(t.data).reshape(t.rows, t.K // V, V)
    else:
        s = _e4m3_decode(q) * t.tensor_scale
        lo, hi = t.data & 15, t.data >> 4
        code = torch.stack([lo, hi], -1).reshape(t.rows, t.K)
        table = torch.tensor(_E2M1)
        vals = (table[(code & 7).long()] * torch.where((code & 8) > 0, -1.0, 1.0)).reshape(t.rows, t.K // V, V)
    return (vals * s.unsqueeze(-1)).reshape(t.rows, t.K)


@nv.traced("gemm_mx")
def gemm_mx(a: MxTensor, b: MxTensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    """a [M, K] x b [N, K] -> [M, N] = a @ b.T, scale factors applied by the tensor core, fp32 accumulation."""
    if a.kind != b.kind or a.K != b.K:
        raise ValueError("operands must share the format and K")
    if not a.data.is_cuda:
        return (dequantize_mx(a) @ dequantize_mx(b).t()).to(out_dtype)
    if b.rows % 8 != 0:
        raise ValueError("N must be a multiple of 8")
    from .gemm import _num_sms
    out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=a.data.device)
    g = MxGemmArgs()
    g.A, g.B, g.sfa, g.sfb = a.data.data_ptr(), b.data.data_ptr(), a.sf.data_ptr(), b.sf.data_ptr()
    g.C, g.ldc = out.data_ptr(), out.stride(0)
    g.M, g.N, g.K = a.rows, b.rows, a.K
    g.out_f32 = int(out_dtype == torch.float32)
    g.alpha = float(a.tensor_scale * b.tensor_scale)
    g.kind = a.kind
    g.status = nv.status_word(a.data.device).data_ptr()
    nv.check(nv.cuda().b200_gemm_mx(C.byref(g), _num_sms(a.data.device), nv.stream_ptr()), "gemm_mx")
    nv.count_launch()
    return out


class MxLinear:
    """Inference Linear with the weight stored block-scaled ([out, in], K = in) and the activations quantised on the fly;
    bias and output in bf16. The tensor-core counterpart of the reference's `QuantizedLinear` (src/quantize.rs:617-700),
    which dequantises the weight to fp32 before a plain matmul."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, kind: str = "mxfp8"):
        self.kind = kind
        self.out_features, self.in_features = weight.shape
        self.weight = quantize_mx(weight, kind)
        self.bias = bias.detach().to(torch.bfloat16) if bias is not None else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        xq = quantize_mx(x.reshape(-1, self.in_features), self.kind)
        y = gemm_mx(xq, self.weight, torch.bfloat16)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)

    __call__ = forward

    def memory_bytes(self) -> int:
        return self.weight.nbytes + (self.bias.numel() * 2 if self.bias is not None else 0)
