"""GEMM front-end: the replacement for rust-nn's `blas::sgemm` (src/blas.rs:104-186).

``gemm(a, b, ...)`` computes ``act(alpha * A @ B^T + bias) [* act'(aux_in)] [+ residual]`` where
``A`` is logically ``[M, K]`` and ``B`` is logically ``[N, K]``. ``a_mn`` / ``b_mn`` say that the
operand is *stored* transposed (``[K, M]`` / ``[K, N]``); no transposed copy is ever made - the
layout goes into the TMA descriptor and the tensor-core matrix descriptor.

On CUDA tensors this always launches the hand-written tcgen05 kernel (csrc/gemm/gemm_sm100.cu).
On CPU tensors it evaluates the same expression with PyTorch in fp32 (the oracle).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from .. import _native as nv

ACT = {"none": 0, "relu": 1, "gelu": 2, "silu": 3, "sigmoid": 4, "tanh": 5}
OUT_BF16, OUT_F32, OUT_F32_ATOMIC, OUT_I32 = 0, 1, 2, 3
GEMM_BF16, GEMM_F32, GEMM_S8S8, GEMM_U8S8, GEMM_E4M3 = 0, 1, 2, 3, 4
_NUM_SMS = {}


def _num_sms(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _NUM_SMS:
        _NUM_SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _NUM_SMS[idx]


def act_ref(x: torch.Tensor, act: str) -> torch.Tensor:
    if act == "relu":
        return torch.relu(x)
    if act == "gelu":
        return torch.nn.functional.gelu(x, approximate="tanh")
    if act == "silu":
        return torch.nn.functional.silu(x)
    if act == "sigmoid":
        return torch.sigmoid(x)
    if act == "tanh":
        return torch.tanh(x)
    return x


def dact_ref(saved: torch.Tensor, act: str) -> torch.Tensor:
    """Derivative of `act` given the saved tensor (pre-activation for gelu/silu, output otherwise)."""
    s = saved.float()
    if act == "relu":
        return (s > 0).float()
    if act == "gelu":
        k0, k1 = 0.7978845608028654, 0.044715
        t = torch.tanh(k0 * (s + k1 * s ** 3))
        return 0.5 * (1 + t) + 0.5 * s * (1 - t * t) * k0 * (1 + 3 * k1 * s * s)
    if act == "silu":
        sg = torch.sigmoid(s)
        return sg * (1 + s * (1 - sg))
    if act == "sigmoid":
        return s * (1 - s)
    if act == "tanh":
        return 1 - s * s
    return torch.ones_like(s)


def gemm_ref(a, b, *, a_mn=False, b_mn=False, bias=None, act="none", residual=None, aux_in=None, dact="none",
             alpha=1.0, out_dtype=None, accumulate_into=None, want_aux=False, row_scale=None, col_scale=None):
    """fp32 PyTorch evaluation of the same expression (used on CPU and as the test oracle)."""
    if out_dtype == torch.int32:          # exact integer accumulation (the igemm contract)
        return (a.to(torch.int64) @ b.to(torch.int64).transpose(-1, -2)).to(torch.int32)
    lowp = a.dtype in (torch.int8, torch.uint8, torch.float8_e4m3fn)
    ft = torch.float64 if lowp else torch.float32
    A = a.to(ft).transpose(-1, -2) if a_mn else a.to(ft)
    B = b.to(ft).transpose(-1, -2) if b_mn else b.to(ft)
    v = (alpha * (A @ B.transpose(-1, -2))).float()
    if row_scale is not None:
        v = v * row_scale.float().reshape(*v.shape[:-1], 1)
    if col_scale is not None:
        v = v * col_scale.float()
    if lowp and out_dtype is None:
        out_dtype = torch.bfloat16
    if bias is not None:
        v = v + (bias.float()[:, None, :] if bias.dim() == 2 else bias.float())   # [batch, N]: one vector per batch
    pre = v
    v = act_ref(v, act)
    if aux_in is not None:
        v = v * dact_ref(aux_in, dact)
    if residual is not None:
        v = v + residual.float()
    if accumulate_into is not None:
        accumulate_into.add_(v.to(accumulate_into.dtype))
        v = accumulate_into
    else:
        v = v.to(out_dtype or a.dtype)
    if want_aux:
        return v, pre.to(torch.bfloat16 if lowp else a.dtype)
    return v


def _as3d(t: torch.Tensor):
    if t.dim() == 2:
        return t.unsqueeze(0)
    if t.dim() == 3:
        return t
    raise ValueError("gemm operands must be 2-D or 3-D")


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Return `t` (3-D view) or a padded copy such that TMA constraints hold:
    innermost stride 1, other strides multiples of 16 bytes, base 16-byte aligned."""
    es = t.element_size()
    q = 16 // es
    ok = t.stride(-1) == 1 and t.stride(-2) % q == 0 and t.data_ptr() % 16 == 0 and t.stride(-2) >= t.shape[-1]
    if ok and t.shape[0] > 1:
        ok = t.stride(0) % q == 0
    if ok:
        return t
    inner = (t.shape[-1] + q - 1) // q * q
    buf = torch.zeros(t.shape[0], t.shape[1], inner, dtype=t.dtype, device=t.device)
    buf[..., : t.shape[-1]].copy_(t)
    return buf[..., : t.shape[-1]]


@nv.traced("gemm")
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias=None, act: str = "none",
         residual=None, aux_in=None, dact: str = "none", want_aux: bool = False, alpha: float = 1.0,
         out_dtype=None, accumulate_into=None, splits: int = 0, bn: int = 0, alpha_t=None, row_scale=None, col_scale=None,
         out=None, m_valid=None, k_valid=None, _prepare: bool = False):
    """See module docstring. Returns C (and the bf16 pre-activation when ``want_aux``). ``out`` (GPU only): write the
    result into this tensor ([M, N] or [batch, M, N], unit inner stride, dtype of the result) instead of a new one.
    ``m_valid`` / ``k_valid`` (int32 [batch] on the device) make a batched product ragged, as the groups of tokens routed
    to each expert are: row tiles of 128 wholly past ``m_valid[b]`` are skipped (those rows of the result are NOT
    written), and the contraction stops at ``k_valid[b]`` rounded up to 128 (rows up to there must hold finite values).

    8-bit operands (int8 x int8, uint8 x int8, float8_e4m3fn x float8_e4m3fn; both K-major) run on the
    tensor cores' integer / fp8 kinds. ``row_scale`` ([M] or [batch, M] fp32) and ``col_scale`` ([N] fp32)
    dequantise in the epilogue before bias and activation; ``out_dtype=torch.int32`` returns the raw
    accumulators of an integer product (rust-nn `igemm`, src/int8.rs:222-314)."""
    if not a.is_cuda:
        if alpha_t is not None:
            alpha = alpha * float(alpha_t)
        r = gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act=act, residual=residual, aux_in=aux_in, dact=dact,
                     alpha=alpha, out_dtype=out_dtype, accumulate_into=accumulate_into, want_aux=want_aux,
                     row_scale=row_scale, col_scale=col_scale)
        # (m_valid / k_valid only skip work whose operands are zero or whose results are never read: nothing to do on CPU)
        if out is not None:
            out.copy_((r[0] if want_aux else r).reshape(out.shape))
            r = (out, r[1]) if want_aux else out
        return r
    lib = nv.cuda()
    kinds = {(torch.bfloat16, torch.bfloat16): GEMM_BF16, (torch.float32, torch.float32): GEMM_F32,
             (torch.int8, torch.int8): GEMM_S8S8, (torch.uint8, torch.int8): GEMM_U8S8,
             (torch.float8_e4m3fn, torch.float8_e4m3fn): GEMM_E4M3}
    if (a.dtype, b.dtype) not in kinds:
        raise TypeError(f"gemm operands must be bf16 x bf16, fp32 x fp32, int8 x int8, uint8 x int8 or e4m3 x e4m3 (got {a.dtype}, {b.dtype})")
    kind = kinds[(a.dtype, b.dtype)]
    is_f32 = kind == GEMM_F32
    lowp = kind >= GEMM_S8S8
    if lowp and (a_mn or b_mn):
        raise ValueError("8-bit GEMM operands must be K-major")
    if is_f32 and (a_mn or b_mn):
        # TF32 tiles are K-major only; 32-bit MN-major operands are transposed by a kernel first
        from .kernels import transpose_last2
        if a_mn:
            a, a_mn = transpose_last2(a), False
        if b_mn:
            b, b_mn = transpose_last2(b), False
    squeeze = a.dim() == 2
    a3, b3 = _tma_ready(_as3d(a)), _tma_ready(_as3d(b))
    batch = a3.shape[0]
    if b3.shape[0] != batch:
        raise ValueError("batch mismatch")
    M, K = (a3.shape[2], a3.shape[1]) if a_mn else (a3.shape[1], a3.shape[2])
    N, Kb = (b3.shape[2], b3.shape[1]) if b_mn else (b3.shape[1], b3.shape[2])
    if K != Kb:
        raise ValueError(f"gemm K mismatch: {K} vs {Kb}")
    dev = a.device
    if accumulate_into is not None:
        out = accumulate_into
        if out.dtype != torch.float32 or not out.is_contiguous():
            raise ValueError("accumulate_into must be a contiguous fp32 tensor")
        out_mode = OUT_F32_ATOMIC
    else:
        odt = out_dtype or (torch.float32 if is_f32 else torch.bfloat16)
        if odt == torch.int32:
            if kind not in (GEMM_S8S8, GEMM_U8S8):
                raise TypeError("an int32 result needs integer operands")
            out_mode = OUT_I32
        else:
            out_mode = OUT_F32 if odt == torch.float32 else OUT_BF16
        if out is not None:
            want = torch.int32 if out_mode == OUT_I32 else torch.float32 if out_mode == OUT_F32 else torch.bfloat16
            if out.dtype != want or out.stride(-1) != 1 or out.numel() != batch * M * N:
                raise ValueError("`out` must have the result's dtype, size and a unit inner stride")
            if splits > 1:
                raise ValueError("`out` and split-K do not go together (split-K accumulates into a zeroed fp32 buffer)")
            splits = splits or 1
    # tile width and split-K
    sms = _num_sms(dev)
    if is_f32:
        bn = 128
    elif lowp:
        bn = 256 if (bn == 256 or (bn == 0 and math.ceil(M / 128) * math.ceil(N / 256) * batch >= sms)) else 128
    elif bn == 0:
        if N <= 64:
            bn = 64
        elif N <= 128:
            bn = 128
        else:
            t256 = math.ceil(M / 128) * math.ceil(N / 256) * batch
            # Few tiles and a long K (weight gradients): split-K fills the machine either way, and the wider tile moves
            # a third less operand traffic from L2 per FLOP (measured 167 -> 113 us on 2048 x 512 x 65536).
            splittable = (splits == 0 and out_mode in (OUT_F32, OUT_F32_ATOMIC) and act == "none" and aux_in is None and not want_aux
                          and N >= 256 and K >= 16 * 64 * max(1, sms // max(t256, 1)))
            bn = 256 if (t256 >= sms or splittable) else 128
    bk = 32 if is_f32 else 128 if lowp else 64
    num_kb = max(1, math.ceil(K / bk))
    tiles = math.ceil(M / 128) * math.ceil(N / bn) * batch
    if splits == 0:
        splits = 1
        if out_mode in (OUT_F32, OUT_F32_ATOMIC) and tiles < sms // 2 and num_kb >= 16 and act == "none" and aux_in is None and not want_aux:
            splits = max(1, min(sms // tiles, num_kb // 8))
    if splits > 1:
        per = math.ceil(num_kb / splits)
        splits = math.ceil(num_kb / per)
    if splits > 1:
        if out_mode == OUT_BF16 or act != "none" or aux_in is not None or want_aux:
            raise ValueError("split-K needs an fp32 output and a linear epilogue")
        out_mode = OUT_F32_ATOMIC
    if out is None:
        shape = (batch, M, N)
        odt = torch.int32 if out_mode == OUT_I32 else torch.float32 if out_mode != OUT_BF16 else torch.bfloat16
        out = torch.zeros(shape, dtype=odt, device=dev) if out_mode == OUT_F32_ATOMIC else torch.empty(shape, dtype=odt, device=dev)
    out3 = out if out.dim() == 3 else out.view(1, M, N) if batch == 1 else out.view(batch, M, N)
    ldc = out3.stride(1)
    aux = torch.empty((batch, M, N), dtype=torch.bfloat16, device=dev) if want_aux else None
    if aux_in is not None:
        aux_in = aux_in.contiguous().view(batch, M, N)
        if aux_in.dtype != torch.bfloat16:
            raise TypeError("aux_in must be bf16")
    if residual is not None:
        residual = residual.reshape(batch, M, N)
        if residual.dtype != torch.bfloat16:
            residual = residual.to(torch.bfloat16)
        if residual.stride(-1) != 1:
            residual = residual.contiguous()
    if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("bias must be fp32 or bf16")

    args = nv.GemmArgs()
    p = args.p
    p.M, p.N, p.K, p.batch, p.splits = M, N, K, batch, splits
    p.C, p.ldc, p.strideC = out3.data_ptr(), ldc, out3.stride(0) if batch > 1 else M * ldc
    p.bias = nv.ptr(bias); p.bias_f32 = 1 if (bias is not None and bias.dtype == torch.float32) else 0
    p.bias_vec_ok = 1 if (bias is not None and bias.data_ptr() % 16 == 0 and bias.is_contiguous() and N % 4 == 0) else 0
    p.strideBias = N if (bias is not None and bias.dim() == 2) else 0      # [batch, N] bias: one vector per batch
    p.residual = nv.ptr(residual)
    p.ldr = residual.stride(1) if residual is not None else 0
    p.strideR = residual.stride(0) if residual is not None else 0
    p.aux_out = nv.ptr(aux); p.aux_in = nv.ptr(aux_in)
    p.alpha = float(alpha); p.alpha_ptr = nv.ptr(alpha_t.float() if alpha_t is not None and alpha_t.dtype != torch.float32 else alpha_t); p.act = ACT[act]; p.dact = ACT[dact]; p.out_mode = out_mode
    es_out = 4 if out_mode != OUT_BF16 else 2
    aux_ok = (aux is None and aux_in is None) or (ldc == N and N % 8 == 0)
    p.vec_ok = 1 if (ldc * es_out % 16 == 0 and out3.data_ptr() % 16 == 0 and (batch == 1 or p.strideC * es_out % 16 == 0) and aux_ok) else 0
    if (aux is not None or aux_in is not None) and ldc != N:
        raise ValueError("aux tensors need a dense output (ldc == N)")
    p.res_vec_ok = 1 if (residual is not None and residual.stride(1) % 8 == 0 and residual.data_ptr() % 16 == 0 and (batch == 1 or residual.stride(0) % 8 == 0)) else 0
    if row_scale is not None:
        row_scale = row_scale.float().contiguous()
        if row_scale.numel() != batch * M:
            raise ValueError("row_scale needs one value per row of A")
    if col_scale is not None:
        col_scale = col_scale.float().contiguous()
        if col_scale.numel() != N:
            raise ValueError("col_scale needs one value per row of B")
    p.row_scale, p.col_scale = nv.ptr(row_scale), nv.ptr(col_scale)
    p.status = nv.status_word(dev).data_ptr()
    for name, t in (("m_valid", m_valid), ("k_valid", k_valid)):
        if t is not None and (t.dtype != torch.int32 or t.numel() != batch or not t.is_cuda):
            raise ValueError(f"{name} must be an int32 device tensor with one entry per batch")
    p.m_valid, p.k_valid = nv.ptr(m_valid), nv.ptr(k_valid)
    args.A, args.lda, args.strideA, args.a_mn = a3.data_ptr(), a3.stride(1), a3.stride(0), int(a_mn)
    args.B, args.ldb, args.strideB, args.b_mn = b3.data_ptr(), b3.stride(1), b3.stride(0), int(b_mn)
    args.M, args.N, args.K, args.batch, args.dtype = M, N, K, batch, kind
    if _prepare:
        # a fused kernel runs this product itself: hand back the filled launch record, the tile width, the results and
        # everything the record points at (kept alive by the caller until the launch has been issued)
        res = out3[0] if (squeeze and out.dim() == 3) else out
        return args, bn, res, (aux[0] if (aux is not None and squeeze) else aux), (a3, b3, bias, residual, aux_in, row_scale, col_scale, m_valid, k_valid, out3)
    rc = lib.b200_gemm_launch(C.byref(args), bn, sms, nv.stream_ptr())
    nv.check(rc, "b200_gemm_launch")
    nv.count_launch()
    res = out3[0] if (squeeze and out.dim() == 3) else out
    if accumulate_into is not None:
        res = accumulate_into
    if want_aux:
        return res, (aux[0] if squeeze else aux)
    return res
