"""Launchers for csrc/quant/quant.cu plus PyTorch restatements of the same arithmetic.

Every function takes the CUDA kernel on CUDA tensors and the restatement on CPU tensors; the
restatements are the oracles of the GPU tests. Rounding is half-away-from-zero, as Rust's
`f32::round` (rust-nn src/int8.rs:42, src/quantize.rs:310).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as nv

_P, _LL, _I, _F = C.c_void_p, C.c_longlong, C.c_int, C.c_float
nv.register_sigs({
    "b200_quant_rows": [_P, _I, _LL, _I, _LL, _P, _LL, _P, _I, _P],
    "b200_quant_group": [_P, _I, _LL, _LL, _I, _P, _P, _P, _P],
    "b200_dequant_group": [_P, _P, _LL, _LL, _I, _P, _I, _P],
    "b200_ternary_quant": [_P, _I, _LL, _I, _P, _P, _P, _P],
    "b200_ternary_unpack": [_P, _LL, _I, _P, _P, _I, _P],
    "b200_ternary_count": [_P, _LL, _P, _P],
    "b200_rotor_quant": [_P, _I, _P, _LL, _I, _I, _F, _P, _P],
    "b200_csr_spmm": [_P, _P, _P, _P, _P, _I, _I, _P],
})

Q_INT8, Q_INT4, Q_NF4, Q_NVFP4, Q_Q4_0, Q_Q8_0 = range(6)

NF4_TABLE = [-1.0, -0.6961928, -0.52507305, -0.3949175, -0.28444138, -0.18477343, -0.091050036, 0.0,
             0.0795803, 0.1609302, 0.2461123, 0.33791524, 0.44070983, 0.562617, 0.72295684, 1.0]
FP4_MAGNITUDES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def round_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


def _isbf(t) -> int:
    return 1 if t.dtype == torch.bfloat16 else 0


def _f32_or_bf16(t):
    return t if t.dtype in (torch.float32, torch.bfloat16) else t.float()


# ------------------------------------------------------------------ per-row int8 / e4m3
def quant_rows(x: torch.Tensor, mode: str = "int8"):
    """Per-row symmetric quantisation of a 2-D tensor: returns (q [rows, cols] int8 | float8_e4m3fn,
    scales [rows] fp32) with x ~= q * scale[:, None]."""
    assert x.dim() == 2
    qmax = 127.0 if mode == "int8" else 448.0
    if not x.is_cuda:
        xf = x.float()
        m = xf.abs().amax(-1)
        scale = torch.where(m > 0, m / qmax, torch.ones_like(m))
        t = xf / scale[:, None]
        if mode == "int8":
            return round_away(t).clamp(-128, 127).to(torch.int8), scale
        return t.clamp(-448, 448).to(torch.float8_e4m3fn), scale
    x = _f32_or_bf16(x)
    if x.stride(-1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8 if mode == "int8" else torch.float8_e4m3fn, device=x.device)
    scales = torch.empty(rows, dtype=torch.float32, device=x.device)
    nv.check(nv.cuda().b200_quant_rows(x.data_ptr(), _isbf(x), rows, cols, x.stride(0), q.data_ptr(), cols, scales.data_ptr(),
                                       0 if mode == "int8" else 1, nv.stream_ptr()), "quant_rows")
    nv.count_launch()
    return q, scales


# ------------------------------------------------------------------ group-wise formats
def _bytes_per_group(gs: int, fmt: int) -> int:
    return gs if fmt in (Q_INT8, Q_Q8_0) else (gs + 1) // 2


def _group_scale_ref(m, fmt):
    one = torch.ones_like(m)
    if fmt in (Q_INT8, Q_Q8_0):
        return torch.where(m > 0, m / 127.0, one)
    if fmt == Q_INT4:
        return torch.where(m > 0, m / 7.0, one)
    if fmt == Q_NF4:
        return torch.where(m > 0, m, one)
    if fmt == Q_NVFP4:
        return torch.where(m > 0, m / 6.0, one)
    s = m / -8.0
    return torch.where(s == 0, one, s)


def _codes_ref(t, fmt):
    if fmt in (Q_INT8, Q_Q8_0):
        return round_away(t).clamp(-128, 127).to(torch.int16) & 0xFF
    if fmt in (Q_INT4, Q_Q4_0):
        return round_away(t).clamp(-8, 7).to(torch.int16) & 0xF
    if fmt == Q_NF4:
        tab = torch.tensor(NF4_TABLE, dtype=torch.float32, device=t.device)
        return (t[..., None] - tab).abs().argmin(-1).to(torch.int16)
    mag = torch.tensor(FP4_MAGNITUDES, dtype=torch.float32, device=t.device)
    best = (t.abs()[..., None] - mag).abs().argmin(-1).to(torch.int16)
    return best | ((t < 0).to(torch.int16) << 3)


def _dequant_codes_ref(c, fmt):
    c = c.to(torch.int32)
    if fmt in (Q_INT8, Q_Q8_0):
        return torch.where(c >= 128, c - 256, c).float()
    if fmt in (Q_INT4, Q_Q4_0):
        return torch.where(c >= 8, c - 16, c).float()
    if fmt == Q_NF4:
        return torch.tensor(NF4_TABLE, dtype=torch.float32, device=c.device)[c.long() & 15]
    mag = torch.tensor(FP4_MAGNITUDES, dtype=torch.float32, device=c.device)[c.long() & 7]
    return torch.where((c & 8) != 0, -mag, mag)


def quant_group_ref(x: torch.Tensor, gs: int, fmt: int):
    flat = x.reshape(-1).float()
    n = flat.numel()
    groups = (n + gs - 1) // gs
    pad = torch.zeros(groups * gs, dtype=torch.float32, device=x.device)
    pad[:n] = flat
    g = pad.view(groups, gs)
    scale = _group_scale_ref(g.abs().amax(-1), fmt)
    codes = _codes_ref(g / scale[:, None], fmt)
    valid = (torch.arange(groups * gs, device=x.device) < n).view(groups, gs)
    codes = torch.where(valid, codes, torch.zeros_like(codes))
    if fmt in (Q_INT8, Q_Q8_0):
        data = codes.reshape(-1)[:n].to(torch.uint8)
    else:
        if gs % 2:
            codes = torch.cat([codes, torch.zeros(groups, 1, dtype=codes.dtype, device=x.device)], 1)
        data = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8).reshape(-1)
        last = n - (groups - 1) * gs
        data = data[: (groups - 1) * ((gs + 1) // 2) + (last + 1) // 2]
    return data.contiguous(), scale.contiguous()


def dequant_group_ref(data, scales, n: int, gs: int, fmt: int, out_dtype=torch.float32):
    i = torch.arange(n, device=data.device)
    g, j = i // gs, i % gs
    if fmt in (Q_INT8, Q_Q8_0):
        c = data[i].to(torch.int32)
    else:
        b = data[g * ((gs + 1) // 2) + j // 2].to(torch.int32)
        c = torch.where(j % 2 == 1, (b >> 4) & 0xF, b & 0xF)
    return (_dequant_codes_ref(c, fmt) * scales[g]).to(out_dtype)


def quant_group(x: torch.Tensor, gs: int, fmt: int):
    """Returns (data uint8, scales fp32[groups]) in the reference's layout."""
    n = x.numel()
    if gs <= 0:
        gs = max(n, 1)
    if not x.is_cuda:
        return quant_group_ref(x, gs, fmt)
    xf = _f32_or_bf16(x).contiguous()
    groups = (n + gs - 1) // gs
    last = n - (groups - 1) * gs
    nbytes = n if fmt in (Q_INT8, Q_Q8_0) else (groups - 1) * ((gs + 1) // 2) + (last + 1) // 2
    # the kernel writes whole pairs, so leave room for one pad byte per group
    data = torch.zeros(max(nbytes, groups * _bytes_per_group(gs, fmt)), dtype=torch.uint8, device=x.device)
    scales = torch.empty(groups, dtype=torch.float32, device=x.device)
    absmax = torch.empty(groups, dtype=torch.int32, device=x.device)
    nv.check(nv.cuda().b200_quant_group(xf.data_ptr(), _isbf(xf), n, gs, fmt, absmax.data_ptr(), scales.data_ptr(), data.data_ptr(),
                                        nv.stream_ptr()), "quant_group")
    nv.count_launch(2)
    return data[:nbytes], scales


def dequant_group(data, scales, n: int, gs: int, fmt: int, out_dtype=torch.float32):
    if not data.is_cuda:
        return dequant_group_ref(data, scales, n, gs, fmt, out_dtype)
    out = torch.empty(n, dtype=out_dtype, device=data.device)
    nv.check(nv.cuda().b200_dequant_group(data.data_ptr(), scales.data_ptr(), n, gs, fmt, out.data_ptr(), 1 if out_dtype == torch.bfloat16 else 0,
                                          nv.stream_ptr()), "dequant_group")
    nv.count_launch()
    return out


# ------------------------------------------------------------------ ternary
def ternary_quant(w: torch.Tensor, rows: int, cols: int):
    """Returns (packed int32[ceil(numel/16)], scales fp32[rows]); code 0 -> 0, 1 -> +1, 2 -> -1."""
    numel = rows * cols
    words = (numel + 15) // 16
    if not w.is_cuda:
        wf = w.reshape(rows, cols).float()
        mean = wf.abs().sum(-1) / max(cols, 1)
        codes = torch.where(wf.abs() < 0.7 * mean[:, None], 0, torch.where(wf > 0, 1, 2)).reshape(-1).to(torch.int64)
        pad = torch.zeros(words * 16, dtype=torch.int64)
        pad[:numel] = codes
        shifts = (torch.arange(16, dtype=torch.int64) * 2)
        packed = (pad.view(words, 16) << shifts).sum(-1)
        packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
        return packed, mean.clamp_min(1e-8)
    wf = _f32_or_bf16(w).contiguous()
    packed = torch.empty(words, dtype=torch.int32, device=w.device)
    mean = torch.empty(rows, dtype=torch.float32, device=w.device)
    scales = torch.empty(rows, dtype=torch.float32, device=w.device)
    nv.check(nv.cuda().b200_ternary_quant(wf.data_ptr(), _isbf(wf), rows, cols, mean.data_ptr(), scales.data_ptr(), packed.data_ptr(),
                                          nv.stream_ptr()), "ternary_quant")
    nv.count_launch(2)
    return packed, scales


def ternary_unpack(packed, numel: int, cols: int, scales=None, out_dtype=torch.float32):
    """{-1, 0, +1} values (times the row scale when `scales` is given), flat [numel]."""
    if not packed.is_cuda:
        i = torch.arange(numel)
        word = packed.to(torch.int64)[i // 16] & 0xFFFFFFFF
        code = (word >> ((i % 16) * 2)) & 3
        v = torch.where(code == 1, 1.0, torch.where(code == 2, -1.0, 0.0))
        if scales is not None:
            v = v * scales[i // cols]
        return v.to(out_dtype)
    out = torch.empty(numel, dtype=out_dtype, device=packed.device)
    nv.check(nv.cuda().b200_ternary_unpack(packed.data_ptr(), numel, cols, nv.ptr(scales), out.data_ptr(), 1 if out_dtype == torch.bfloat16 else 0,
                                           nv.stream_ptr()), "ternary_unpack")
    nv.count_launch()
    return out


def ternary_counts(packed, numel: int):
    """(+1 count, -1 count, 0 count)."""
    if not packed.is_cuda:
        v = ternary_unpack(packed, numel, max(numel, 1))
        return int((v == 1).sum()), int((v == -1).sum()), int((v == 0).sum())
    counts = torch.empty(3, dtype=torch.int64, device=packed.device)
    nv.check(nv.cuda().b200_ternary_count(packed.data_ptr(), numel, counts.data_ptr(), nv.stream_ptr()), "ternary_count")
    nv.count_launch()
    c = counts.tolist()
    return c[0], c[1], c[2]


# ------------------------------------------------------------------ RotorQuant
def rotor_quant_ref(x, rot, dim: int, qmax: float):
    groups = rot.shape[0]
    rows = x.numel() // dim
    pad = torch.zeros(rows, groups * 3, dtype=torch.float32, device=x.device)
    pad[:, :dim] = x.reshape(rows, dim).float()
    v = pad.view(rows, groups, 3)
    R = rot.view(groups, 3, 3).float()
    rv = torch.einsum("gab,rgb->rga", R, v)
    m = rv.abs().amax(-1, keepdim=True)
    scale = m / qmax
    q = round_away(rv / scale.clamp_min(1e-38)).clamp(-qmax, qmax) * scale
    out = torch.einsum("gab,rga->rgb", R, q)
    out = torch.where(m < 1e-12, v, out)
    return out.reshape(rows, groups * 3)[:, :dim].reshape(x.shape).to(x.dtype)


def rotor_quant(x, rot, dim: int, qmax: float):
    if not x.is_cuda:
        return rotor_quant_ref(x, rot, dim, qmax)
    xf = _f32_or_bf16(x).contiguous()
    out = torch.empty_like(xf)
    rows = xf.numel() // dim
    nv.check(nv.cuda().b200_rotor_quant(xf.data_ptr(), _isbf(xf), rot.data_ptr(), rows, dim, rot.shape[0], float(qmax), out.data_ptr(),
                                        nv.stream_ptr()), "rotor_quant")
    nv.count_launch()
    return out.to(x.dtype)


# ------------------------------------------------------------------ CSR SpMM
def csr_spmm(values, col_idx, row_ptr, b, m: int, n: int):
    """C[m, n] = S * B with S in CSR (fp32 values, int32 indices), B [k, n] fp32 row-major."""
    if not values.is_cuda:
        out = torch.zeros(m, n, dtype=torch.float32)
        rows = torch.repeat_interleave(torch.arange(m), (row_ptr[1:] - row_ptr[:-1]).long())
        out.index_add_(0, rows, values[:, None] * b.reshape(-1, n)[col_idx.long()])
        return out
    b = b.float().contiguous()
    out = torch.empty(m, n, dtype=torch.float32, device=values.device)
    nv.check(nv.cuda().b200_csr_spmm(values.data_ptr(), col_idx.data_ptr(), row_ptr.data_ptr(), b.data_ptr(), out.data_ptr(), m, n,
                                     nv.stream_ptr()), "csr_spmm")
    nv.count_launch()
    return out
