"""Tensor parallelism over NVLink peer memory: the two GEMM + collective fusions of a sharded MLP /
attention block (the reference has no tensor parallelism; its only multi-worker path is the
simulated gradient all-reduce, rust-nn src/distributed.rs:54-124).

  `all_gather_gemm`     Y[M, N_local] = gather_rows(X_shard) @ W_shard^T  - column-parallel Linear after a
                        sequence-sharded activation. Gather CTAs push this rank's row blocks of X into every
                        peer's staging copy and raise a flag per 128-row block there; the GEMM's TMA producers
                        wait on their local flags, so arrived rows multiply while later ones are in flight.
  `gemm_reduce_scatter` Y_shard[M/world, N] = sum_r X[:, K_r] @ W[:, K_r]^T   - row-parallel Linear. Each
                        rank's epilogue stores its partial tiles into the owner's slot buffer (plain peer
                        stores), one cross-rank handshake, then every CTA sums the slots of the local rows
                        (+ residual) - all in one kernel (csrc/gemm/gemm_sm100.cu, `TpParams`).

Both run as ONE kernel per rank and per call; all waits are bounded by `wait_seconds` and end in the
status word. `backend="nccl"` is the baseline (all_gather / reduce_scatter + the plain GEMM) the fused
kernels are measured against, and the path CPU (gloo) ranks take.
"""
from __future__ import annotations

import ctypes as C
import os
import math
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import gemm as G

TP_MAX_WORLD = 8
TP_AG_GEMM, TP_GEMM_RS = 1, 2
BM = 128


class TpParams(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("rank", C.c_int), ("world", C.c_int), ("copy_ctas", C.c_int),
        ("blocks_per_rank", C.c_int), ("epoch_ptr", C.c_void_p), ("wait_cycles", C.c_longlong),
        ("stage_peer", C.c_void_p * TP_MAX_WORLD), ("ready_peer", C.c_void_p * TP_MAX_WORLD),
        ("slots_peer", C.c_void_p * TP_MAX_WORLD), ("out", C.c_void_p), ("go", C.c_void_p),
        ("flags", C.c_void_p * TP_MAX_WORLD), ("done_ctr", C.c_void_p),
    ]


AR_MAX_WORLD, AR_MAX_CTAS = 8, 64


class AllReduceArgs(C.Structure):
    _fields_ = [("in_sym", C.c_void_p * AR_MAX_WORLD), ("red_sym", C.c_void_p * AR_MAX_WORLD), ("flags", C.c_void_p * AR_MAX_WORLD),
                ("inp", C.c_void_p), ("out", C.c_void_p), ("numel", C.c_longlong), ("rank", C.c_int), ("world", C.c_int),
                ("in_bf16", C.c_int), ("wait_cycles", C.c_longlong), ("status", C.c_void_p), ("words", C.c_void_p)]


nv.register_sigs({"b200_gemm_tp_launch": [C.POINTER(nv.GemmArgs), C.POINTER(TpParams), C.c_int, C.c_int, C.c_void_p],
                  "b200_allreduce_bf16": [C.POINTER(AllReduceArgs), C.c_int, C.c_void_p]})


class TPContext:
    """Symmetric buffers and flags of one tensor-parallel group, sized for the largest call it will serve."""

    def __init__(self, max_rows: int, max_k: int, max_n: int, device=None, group=None, backend: str = "fused",
                 wait_seconds: float = 2.0, copy_ctas: int = 0, max_allreduce_numel: int = 0):
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.backend = backend if self.device.type == "cuda" else "nccl"
        self.max_rows, self.max_k, self.max_n = max_rows, max_k, max_n
        # gather CTAs of the all-gather -> GEMM kernel, 0: chosen per call. Measured: 32 of the 148 is best on 2 GPUs; on 8 GPUs
        # 64 is best while the push is small (59 MB: 0.185 ms against 0.201 with 32: latency, more chains in flight) and 32 once
        # it is large (940 MB: 1.82 ms against 2.08 with 64: the links are full either way and the tiles want the SMs)
        env_c = int(os.environ.get("B200NN_TP_COPY_CTAS", "0"))
        self.copy_ctas = copy_ctas if copy_ctas > 0 else env_c
        if self.backend == "fused":
            from .ddp import SymmetricBuffer
            if max_rows % (self.world * BM) != 0:
                raise ValueError(f"rows ({max_rows}) must be a multiple of world * {BM}")
            self.rows_per_rank = max_rows // self.world
            dev = self.device
            # all-gather staging [2][M, K]: calls alternate between the halves, so the gathered rows of a call stay
            # readable (e.g. for the weight gradient that follows) until the call after the next one
            self.stage = SymmetricBuffer(2 * max_rows * max_k, torch.bfloat16, dev, self.group)
            self.ag_calls = 0
            # `keep_gathered` copies a call's gathered rows out of the staging half on this stream, beside whatever the
            # main stream runs next; the next all-gather call (or the consumer of the copy) waits for it
            self.side = torch.cuda.Stream(dev)
            self._copy_done = None
            self.slots = SymmetricBuffer(2 * self.world * self.rows_per_rank * max_n, torch.bfloat16, dev, self.group)
            self.flags = SymmetricBuffer(2 * TP_MAX_WORLD + max_rows // BM, torch.int32, dev, self.group)   # handshake words, then ready[m_blocks]
            # go, done_ctr, call epoch. The epoch is a DEVICE word that each call's last CTA advances, so a captured launch
            # replays with a fresh epoch; it is shared by both kernels. Reuse rules of the buffers:
            #  * gather staging: an all-gather call ends with a cross-rank handshake ("my GEMM no longer reads my staging
            #    copy"), so when it returns every rank may be pushed into again. The two halves exist only so that the
            #    gathered rows of a call stay readable for the weight-gradient GEMM until the call after the next one.
            #  * reduce-scatter slots: selected by epoch & 1. Two reduce-scatter calls in a row get different halves; with
            #    any call in between, that call's handshake orders the second store after the first sum. A rank can be at
            #    most one call ahead of its slowest peer, because every call waits for all ranks' flags of that epoch.
            self.local = torch.zeros(8, dtype=torch.int32, device=dev)
            self.ar_numel = (max_allreduce_numel + 63) // 64 * 64
            if self.ar_numel:
                self.ar_in = SymmetricBuffer(self.ar_numel, torch.float32, dev, self.group)
                self.ar_red = SymmetricBuffer(self.ar_numel, torch.bfloat16, dev, self.group)
                self.ar_flags = SymmetricBuffer(3 * AR_MAX_WORLD * AR_MAX_CTAS, torch.int32, dev, self.group)
                self.ar_words = torch.zeros(4, dtype=torch.int32, device=dev)
            self.clock_hz = torch.cuda.get_device_properties(dev).clock_rate * 1000
            self.wait_cycles = int(wait_seconds * self.clock_hz)
            self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
            dist.barrier(self.group)
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ all-gather -> GEMM
    def ag_input(self, rows_local: int, k: int) -> torch.Tensor:
        """[rows_local, k] bf16 view of this rank's rows inside the gather staging buffer: write the local
        activation shard here (peers read it in place)."""
        if rows_local * self.world > self.max_rows or k > self.max_k:
            raise ValueError("call exceeds the context's capacity")
        return self._stage_view(self.ag_calls & 1, rows_local, k)[self.rank * rows_local:(self.rank + 1) * rows_local]

    def _stage_view(self, half: int, rows_local: int, k: int) -> torch.Tensor:
        m = rows_local * self.world
        off = half * self.max_rows * self.max_k
        return self.stage.tensor[off: off + m * k].view(m, k)

    def _gather_ctas(self, rows_local: int, k: int) -> int:
        if self.copy_ctas > 0:
            return self.copy_ctas
        pushed = rows_local * k * 2 * (self.world - 1)
        return 32 if (self.world <= 2 or pushed >= (256 << 20)) else 64

    def _tp(self, mode: int, rows_local: int, k: int = 0) -> TpParams:
        tp = TpParams()
        tp.mode, tp.rank, tp.world = mode, self.rank, self.world
        tp.copy_ctas = self._gather_ctas(rows_local, k) if (mode == TP_AG_GEMM and self.world > 1) else 0
        tp.blocks_per_rank = rows_local // BM
        tp.epoch_ptr, tp.wait_cycles = self.local.data_ptr() + 8, self.wait_cycles
        tp.go = self.local.data_ptr()
        tp.done_ctr = self.local.data_ptr() + 4
        for r in range(self.world):
            tp.flags[r] = self.flags.ptrs[r]
            tp.ready_peer[r] = self.flags.ptrs[r] + 4 * 2 * TP_MAX_WORLD
        return tp

    def all_gather_gemm(self, x_shard: torch.Tensor, w_shard: torch.Tensor, bias=None, act: str = "none", want_aux: bool = False,
                        return_gathered: bool = False):
        """x_shard [rows_local, K] (this rank's rows; if it is not already `ag_input(...)` it is copied there),
        w_shard [N_local, K] -> act(gather(x) @ w_shard^T + bias) [rows_local * world, N_local] bf16.
        `return_gathered` appends gather(x) [M, K] to the result: on the fused path a view of the staging half of this
        call, valid until the call after the next one on this context."""
        rows_local, k = x_shard.shape
        n = w_shard.shape[0]
        m = rows_local * self.world
        if self.backend != "fused":
            xs = [torch.empty_like(x_shard) for _ in range(self.world)]
            dist.all_gather(xs, x_shard.contiguous(), group=self.group)
            xg = torch.cat(xs, 0)
            res = G.gemm(xg, w_shard, bias=bias, act=act, want_aux=want_aux)
            if not return_gathered:
                return res
            return (*res, xg) if want_aux else (res, xg)
        if rows_local % BM != 0 or k % 8 != 0 or n % 8 != 0:
            raise ValueError("fused all_gather_gemm needs rows_local % 128 == 0 and K, N % 8 == 0")
        self.join_copy()                 # peers push into the other half's predecessor once this call's kernel has run
        mine = self.ag_input(rows_local, k)
        if x_shard.data_ptr() != mine.data_ptr():
            mine.copy_(x_shard)
        half = self.ag_calls & 1
        self.ag_calls += 1
        tp = self._tp(TP_AG_GEMM, rows_local, k)
        for r in range(self.world):
            tp.stage_peer[r] = self.stage.ptrs[r] + half * self.max_rows * self.max_k * 2
        out = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
        aux = torch.empty(m, n, dtype=torch.bfloat16, device=self.device) if want_aux else None
        self._launch(tp, self._stage_view(half, rows_local, k), w_shard, m, n, k, out, bias, act, None, aux)
        res = (out, aux) if want_aux else (out,)
        if return_gathered:
            res = (*res, self._stage_view(half, rows_local, k))
        return res if len(res) > 1 else res[0]

    def join_copy(self) -> None:
        """Main stream waits for the outstanding `keep_gathered` copy, if any."""
        if getattr(self, "_copy_done", None) is not None:
            torch.cuda.current_stream(self.device).wait_event(self._copy_done)
            self._copy_done = None

    def keep_gathered(self, xg: torch.Tensor):
        """A private copy of a call's gathered rows (a view of a staging half, which the call after the next one
        overwrites) for the backward pass. On the fused path the copy runs on a side stream, so the 2 x M x K bytes move
        while the main stream computes; returns (copy, event to wait for before reading it or None)."""
        if self.backend != "fused":
            return xg, None              # a fresh tensor already (torch.cat of the gathered shards)
        keep = torch.empty_like(xg)
        main = torch.cuda.current_stream(self.device)
        fork = torch.cuda.Event()
        fork.record(main)
        self.side.wait_event(fork)
        with torch.cuda.stream(self.side):
            keep.copy_(xg)
            done = torch.cuda.Event()
            done.record(self.side)
        self._copy_done = done
        return keep, done

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, bias=None, residual=None) -> torch.Tensor:
        """x [M, K_local], w [N, K_local] (this rank's K slice) -> rows [rank * M/world, (rank+1) * M/world) of
        sum over ranks of x @ w^T (+ bias, + residual [M/world, N])."""
        m, k = x.shape
        n = w.shape[0]
        rows_local = m // self.world
        if self.backend != "fused":
            part = G.gemm(x, w, bias=bias if self.rank == 0 else None, out_dtype=torch.float32)
            outs = torch.empty(rows_local, n, dtype=torch.float32, device=x.device)
            if x.is_cuda:
                dist.reduce_scatter_tensor(outs, part.contiguous(), group=self.group)
            else:
                dist.all_reduce(part, group=self.group)
                outs = part[self.rank * rows_local:(self.rank + 1) * rows_local]
            if residual is not None:
                outs = outs + residual.float()
            return outs.to(torch.bfloat16)
        if m != self.max_rows and (m % (self.world * BM) != 0):
            raise ValueError("fused gemm_reduce_scatter needs M % (world * 128) == 0")
        if m * n // self.world > self.rows_per_rank * self.max_n or k % 8 != 0 or n % 8 != 0:
            raise ValueError("call exceeds the context's capacity or K, N % 8 != 0")
        tp = self._tp(TP_GEMM_RS, rows_local)
        for r in range(self.world):
            tp.slots_peer[r] = self.slots.ptrs[r]
        out = torch.empty(rows_local, n, dtype=torch.bfloat16, device=self.device)
        tp.out = out.data_ptr()
        if residual is not None:
            residual = residual.to(torch.bfloat16).contiguous()
        dummy = torch.empty(0, dtype=torch.bfloat16, device=self.device)
        self._launch(tp, x.contiguous(), w, m, n, k, dummy, bias if self.rank == 0 else None, "none", residual, None)
        return out

    # ------------------------------------------------------------------ small all-reduce (replicated activations)
    def all_reduce(self, part: torch.Tensor) -> torch.Tensor:
        """Sum of `part` (fp32 or bf16, same shape on every rank) over the group, as bf16. One two-shot kernel over peer
        memory (csrc/comm/allreduce.cu); every rank receives identical bits."""
        if self.backend != "fused":
            t = part.float().contiguous()
            if self.world > 1:
                t = t.clone()
                dist.all_reduce(t, group=self.group)
            return t.to(torch.bfloat16)
        n = part.numel()
        if n > self.ar_numel or n % (8 * self.world) != 0:
            raise ValueError(f"all_reduce of {n} elements: the context holds {self.ar_numel} and needs a multiple of {8 * self.world}")
        if part.dtype not in (torch.float32, torch.bfloat16):
            part = part.float()
        part = part.contiguous()
        out = torch.empty(part.shape, dtype=torch.bfloat16, device=self.device)
        a = AllReduceArgs()
        for r in range(self.world):
            a.in_sym[r], a.red_sym[r], a.flags[r] = self.ar_in.ptrs[r], self.ar_red.ptrs[r], self.ar_flags.ptrs[r]
        a.inp, a.out, a.numel = part.data_ptr(), out.data_ptr(), n
        a.rank, a.world, a.in_bf16 = self.rank, self.world, int(part.dtype == torch.bfloat16)
        a.wait_cycles, a.status, a.words = self.wait_cycles, nv.status_word(self.device).data_ptr(), self.ar_words.data_ptr()
        grid = max(1, min(AR_MAX_CTAS, n // (8 * self.world * 512)))
        nv.check(nv.cuda().b200_allreduce_bf16(C.byref(a), grid, nv.stream_ptr()), "allreduce_bf16")
        nv.count_launch()
        self._keep_ar = (part, out)
        return out

    def _launch(self, tp, a, b, m, n, k, out, bias, act, residual, aux):
        args = nv.GemmArgs()
        p = args.p
        p.M, p.N, p.K, p.batch, p.splits = m, n, k, 1, 1
        p.C, p.ldc, p.strideC = out.data_ptr() if out.numel() else 0, n, m * n
        if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
            bias = bias.float()
        p.bias = nv.ptr(bias); p.bias_f32 = 1 if (bias is not None and bias.dtype == torch.float32) else 0
        p.bias_vec_ok = 1 if (bias is not None and bias.data_ptr() % 16 == 0 and n % 4 == 0) else 0
        p.strideBias = 0
        p.residual = nv.ptr(residual); p.ldr = n if residual is not None else 0; p.strideR = 0
        p.aux_out = nv.ptr(aux); p.aux_in = 0
        p.alpha, p.alpha_ptr, p.act, p.dact, p.out_mode = 1.0, 0, G.ACT[act], 0, G.OUT_BF16
        p.vec_ok, p.res_vec_ok = 1, 1
        p.row_scale, p.col_scale = 0, 0
        p.status = nv.status_word(self.device).data_ptr()
        b = b if b.stride(-1) == 1 else b.contiguous()
        args.A, args.lda, args.strideA, args.a_mn = a.data_ptr(), a.stride(0), 0, 0
        args.B, args.ldb, args.strideB, args.b_mn = b.data_ptr(), b.stride(0), 0, 0
        args.M, args.N, args.K, args.batch, args.dtype = m, n, k, 1, G.GEMM_BF16
        bn = 256 if math.ceil(m / 128) * math.ceil(n / 256) >= self.sms else 128
        rc = nv.cuda().b200_gemm_tp_launch(C.byref(args), C.byref(tp), bn, self.sms, nv.stream_ptr())
        nv.check(rc, "b200_gemm_tp_launch")
        nv.count_launch()
        self._keep = (a, b, bias, residual, out, aux)          # alive until the next call on this context


# ------------------------------------------------------------------------------------------------------------
# Differentiable sharded layers. The backward of each fused op is the OTHER fused op:
#   column-parallel  Y = gather(X_s) W_s^T     dX_s = reduce_scatter(dY W_s)        dW_s = dY^T gather(X_s)
#   row-parallel     Z_s = reduce_scatter(H W_s^T)   dH = gather(dZ_s) W_s            dW_s = gather(dZ_s)^T H
# so a sharded MLP trains with four fused GEMM + collective kernels and two local weight-gradient GEMMs per step.
class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, b, tpc, act):
        from ..ops.functional import compute_weight
        W = compute_weight(w, x_shard)
        bias = b.detach() if b is not None else None
        if act in ("gelu", "silu"):
            y, pre, xg = tpc.all_gather_gemm(x_shard, W, bias=bias, act=act, want_aux=True, return_gathered=True)
        else:
            y, xg = tpc.all_gather_gemm(x_shard, W, bias=bias, act=act, return_gathered=True)
            pre = y if act == "relu" else None
        # the gathered input is needed for the weight gradient long after the staging half has been reused
        need = any(ctx.needs_input_grad[:3])          # False under no_grad: nothing is kept then
        keep, ctx.keep_done = tpc.keep_gathered(xg) if need else (torch.empty(0), None)
        ctx.save_for_backward(keep, w, b if b is not None else torch.empty(0), pre if pre is not None else torch.empty(0))
        ctx.tpc, ctx.act = tpc, act
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import kernels as K
        from ..ops.functional import compute_weight
        xg, w, b, pre = ctx.saved_tensors
        tpc, act = ctx.tpc, ctx.act
        if ctx.keep_done is not None:
            torch.cuda.current_stream(dy.device).wait_event(ctx.keep_done)
            if tpc._copy_done is ctx.keep_done:
                tpc._copy_done = None
        dy = dy.contiguous()
        db = None
        if act != "none":
            dy, db = K.dact_colsum(dy.clone(), pre, act, want_bias_grad=b.numel() > 0)
        elif b.numel() > 0:
            db = K.colsum(dy)
        dw = G.gemm(dy, xg, a_mn=True, b_mn=True, out_dtype=torch.float32)                  # [N_local, K]
        wt = compute_weight(w, dy).t().contiguous()                                         # [K, N_local]
        dx = tpc.gemm_reduce_scatter(dy, wt)                                                # [rows_local, K]
        return dx, dw.to(w.dtype), (db.to(b.dtype) if db is not None and b.numel() > 0 else None), None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, b, residual, tpc):
        from ..ops.functional import compute_weight
        z = tpc.gemm_reduce_scatter(h, compute_weight(w, h), bias=b.detach() if b is not None else None, residual=residual)
        ctx.save_for_backward(h, w, b if b is not None else torch.empty(0))
        ctx.tpc, ctx.has_res = tpc, residual is not None
        return z

    @staticmethod
    def backward(ctx, dz):
        from ..ops import kernels as K
        from ..ops.functional import compute_weight
        h, w, b = ctx.saved_tensors
        tpc = ctx.tpc
        dz = dz.contiguous()
        wt = compute_weight(w, dz).t().contiguous()                                         # [K_local, N]
        dh, dzg = tpc.all_gather_gemm(dz, wt, return_gathered=True)                         # [M, K_local], gather(dz) [M, N]
        dw = G.gemm(dzg, h, a_mn=True, b_mn=True, out_dtype=torch.float32)                  # [N, K_local]
        db = K.colsum(dzg).to(b.dtype) if b.numel() > 0 else None                           # replicated bias: every rank sums all rows
        return dh, dw.to(w.dtype), db, (dz if ctx.has_res else None), None


class _RowParallelAllReduceFn(torch.autograd.Function):
    """y = all_reduce(h W_s^T): row-parallel Linear whose (narrow) output every rank needs in full. The backward
    all-reduces the incoming gradient, because every rank consumed y in its own computation."""

    @staticmethod
    def forward(ctx, h, w, tpc):
        from ..ops.functional import compute_weight
        part = G.gemm(h, compute_weight(w, h), out_dtype=torch.float32)
        ctx.save_for_backward(h, w)
        ctx.tpc = tpc
        return tpc.all_reduce(part)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.functional import _wgrad, compute_weight
        h, w = ctx.saved_tensors
        g = ctx.tpc.all_reduce(dy.contiguous())
        dh = G.gemm(g, compute_weight(w, g), b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(g, h, w) if ctx.needs_input_grad[1] else None
        return dh, dw, None


class _SplitColsFn(torch.autograd.Function):
    """(x[:, :n], x[:, n:]) as views; the backward writes both gradients into one buffer (two strided copies) where
    autograd's own slice backward would fill two zero matrices of x's size, copy into them and add them."""

    @staticmethod
    def forward(ctx, x, n):
        ctx.n, ctx.shape, ctx.dt = n, x.shape, x.dtype
        return x[:, :n], x[:, n:]

    @staticmethod
    def backward(ctx, g1, g2):
        dev = (g1 if g1 is not None else g2).device
        out = torch.empty(ctx.shape, dtype=ctx.dt, device=dev)
        for g, sl in ((g1, out[:, :ctx.n]), (g2, out[:, ctx.n:])):
            if g is None:
                sl.zero_()
            else:
                sl.copy_(g)
        return out, None


def split_cols(x: torch.Tensor, n: int):
    return _SplitColsFn.apply(x, n)


def row_parallel_all_reduce(h: torch.Tensor, w: torch.Tensor, tpc: "TPContext") -> torch.Tensor:
    return _RowParallelAllReduceFn.apply(h, w, tpc)


def column_parallel(x_shard, w, b, tpc, act="none"):
    return _ColumnParallelFn.apply(x_shard, w, b, tpc, act)


def row_parallel(h, w, b, residual, tpc):
    return _RowParallelFn.apply(h, w, b, residual, tpc)


class _ScaleGradFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, s):
        ctx.s = s
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.s, None


def scale_grad(x: torch.Tensor, s: float) -> torch.Tensor:
    """Identity whose backward multiplies the gradient by `s` (a rank's share of a loss that is a mean over ranks)."""
    return _ScaleGradFn.apply(x, s)


class ColumnParallelLinear:
    """Linear whose OUTPUT features are sharded: this rank holds rows [rank * N/world, (rank + 1) * N/world) of the
    weight. Input: this rank's rows of a row-sharded activation [rows_local, K]; output: all rows, local features
    [rows_local * world, N/world]. `full_weight` / `full_bias`, when given, are sliced (same values on every rank)."""

    def __init__(self, in_features: int, out_features: int, tpc: TPContext, bias: bool = True, act: str = "none",
                 full_weight: Optional[torch.Tensor] = None, full_bias: Optional[torch.Tensor] = None, init_std: float = 0.02):
        if out_features % tpc.world:
            raise ValueError("out_features must divide by the tensor-parallel world size")
        n_local = out_features // tpc.world
        lo = tpc.rank * n_local
        dev = tpc.device
        if full_weight is None:
            g = torch.Generator().manual_seed(1234)
            full_weight = torch.randn(out_features, in_features, generator=g) * init_std
        self.weight = full_weight[lo:lo + n_local].detach().clone().to(dev, torch.float32).requires_grad_(True)
        self.bias = None
        if bias:
            fb = full_bias if full_bias is not None else torch.zeros(out_features)
            self.bias = fb[lo:lo + n_local].detach().clone().to(dev, torch.float32).requires_grad_(True)
        self.tpc, self.act = tpc, act

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def __call__(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _ColumnParallelFn.apply(x_shard, self.weight, self.bias, self.tpc, self.act)


class RowParallelLinear:
    """Linear whose INPUT features are sharded: this rank holds columns [rank * K/world, ...) of the weight. Input:
    all rows, local features [M, K/world]; output: this rank's rows of the full sum [M / world, N] (+ bias, + this
    rank's rows of a residual)."""

    def __init__(self, in_features: int, out_features: int, tpc: TPContext, bias: bool = True,
                 full_weight: Optional[torch.Tensor] = None, full_bias: Optional[torch.Tensor] = None, init_std: float = 0.02):
        if in_features % tpc.world:
            raise ValueError("in_features must divide by the tensor-parallel world size")
        k_local = in_features // tpc.world
        lo = tpc.rank * k_local
        dev = tpc.device
        if full_weight is None:
            g = torch.Generator().manual_seed(4321)
            full_weight = torch.randn(out_features, in_features, generator=g) * init_std
        self.weight = full_weight[:, lo:lo + k_local].detach().clone().to(dev, torch.float32).requires_grad_(True)
        self.bias = None
        if bias:
            fb = full_bias if full_bias is not None else torch.zeros(out_features)
            self.bias = fb.detach().clone().to(dev, torch.float32).requires_grad_(True)
        self.tpc = tpc

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def __call__(self, h: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return _RowParallelFn.apply(h, self.weight, self.bias, residual, self.tpc)


class TensorParallelMLP:
    """x_s + W2 act(W1 gather(x_s)) on row-sharded activations: all-gather -> GEMM (+bias, activation), then
    GEMM -> reduce-scatter (+bias, +residual). Forward and backward are four fused kernels and two local GEMMs."""

    def __init__(self, d_model: int, hidden: int, tpc: TPContext, act: str = "gelu", w1=None, b1=None, w2=None, b2=None):
        self.up = ColumnParallelLinear(d_model, hidden, tpc, act=act, full_weight=w1, full_bias=b1)
        self.down = RowParallelLinear(hidden, d_model, tpc, full_weight=w2, full_bias=b2)

    def parameters(self):
        return self.up.parameters() + self.down.parameters()

    def __call__(self, x_shard: torch.Tensor, residual: bool = True) -> torch.Tensor:
        return self.down(self.up(x_shard), x_shard if residual else None)
