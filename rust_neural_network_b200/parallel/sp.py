"""Sequence (context) parallelism for linear attention: every rank owns a contiguous slice of the
sequence and the ranks exchange only the [d x (d_v + 8)] KV states - O(d^2) per head instead of the
O(S d) keys and values a softmax-attention ring would move. The reference scales sequence length only
algorithmically (rust-nn src/linear_attention.rs:110-300) and has no multi-worker attention.

`SPContext.exclusive_prefix(total)` returns, on rank r, the sum of `total` over ranks < r (differentiable:
the backward is the mirror-image suffix exchange); `all_sum(total)` the sum over all ranks. Both are one
kernel (csrc/comm/state_exchange.cu): publish into peer-mapped memory, flag handshake, peer loads, second
handshake. CPU (gloo) ranks and `backend="nccl"` use an all-gather of the states instead.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist
from torch.autograd import Function

from .. import _native as nv

SX_MAX_WORLD, SX_MAX_CTAS = 8, 64


class StateExchangeArgs(C.Structure):
    _fields_ = [("slot", C.c_void_p * SX_MAX_WORLD), ("flags", C.c_void_p * SX_MAX_WORLD), ("inp", C.c_void_p), ("out", C.c_void_p),
                ("numel", C.c_longlong), ("rank", C.c_int), ("world", C.c_int), ("mode", C.c_int), ("epoch", C.c_uint32),
                ("wait_cycles", C.c_longlong), ("status", C.c_void_p), ("words", C.c_void_p)]


nv.register_sigs({"b200_state_exchange": [C.POINTER(StateExchangeArgs), C.c_int, C.c_void_p], "b200_state_exchange_flag_words": []})

LOWER, HIGHER, ALL = 0, 1, 2


class _ExchangeFn(Function):
    @staticmethod
    def forward(ctx, total, sp, mode):
        ctx.sp, ctx.mode = sp, mode
        return sp._exchange(total, mode)

    @staticmethod
    def backward(ctx, g):
        back = {LOWER: HIGHER, HIGHER: LOWER, ALL: ALL}[ctx.mode]
        return ctx.sp._exchange(g.contiguous(), back), None, None


class SPContext:
    def __init__(self, max_numel: int, device=None, group=None, backend: str = "fused", wait_seconds: float = 2.0, grid: int = 32):
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.backend = backend if self.device.type == "cuda" else "nccl"
        self.max_numel = (max_numel + 3) // 4 * 4
        self.grid = min(grid, SX_MAX_CTAS)
        if self.backend == "fused":
            from .ddp import SymmetricBuffer
            self.slot = SymmetricBuffer(self.max_numel, torch.float32, self.device, self.group)
            self.flags = SymmetricBuffer(2 * SX_MAX_WORLD * SX_MAX_CTAS, torch.int32, self.device, self.group)
            self.words = torch.zeros(4, dtype=torch.int32, device=self.device)     # call epoch + retired-CTA counter, on the device
            self.wait_cycles = int(wait_seconds * torch.cuda.get_device_properties(self.device).clock_rate * 1000)
            dist.barrier(self.group)
            torch.cuda.synchronize()

    def fill_exchange(self, sx, bh: int, st: int, direction: int, role: int) -> torch.Tensor:
        """Fill the `LaExchange` block of a linear-attention launch: the kernels of csrc/attention/linattn_sm100.cu then
        publish (role 1) / pull (role 2) the slice totals of `bh` (batch x head) states of `st` floats themselves.
        One set of buffers per direction (0: forward states flow to higher ranks, 1: backward states to lower ranks),
        allocated on first use - collectively, so every rank must make the same calls. Returns the local buffer the
        consume pass leaves its summed state in."""
        if self.backend != "fused":
            raise RuntimeError("the in-kernel exchange needs the peer-memory backend")
        if not hasattr(self, "_la"):
            self._la = {}
        ent = self._la.get(direction)
        if ent is None or ent["bh"] < bh or ent["st"] != st:
            if ent is not None:
                raise ValueError("the exchange buffers of this context were sized for a smaller batch x heads or another head size")
            from .ddp import SymmetricBuffer
            ent = {"bh": bh, "st": st,
                   "state": SymmetricBuffer(2 * bh * st, torch.float32, self.device, self.group, name=f"la_state{direction}"),
                   "flags": SymmetricBuffer(self.world * bh, torch.int32, self.device, self.group, name=f"la_flags{direction}"),
                   "acks": SymmetricBuffer(self.world * bh, torch.int32, self.device, self.group, name=f"la_acks{direction}"),
                   "prefix": torch.zeros(bh * st, dtype=torch.float32, device=self.device),
                   "words": torch.zeros(2, dtype=torch.int32, device=self.device)}
            dist.barrier(self.group)
            torch.cuda.synchronize()
            self._la[direction] = ent
        if ent["bh"] != bh:
            raise ValueError("batch x heads must stay the same for one context (the flag arrays are indexed by it)")
        for r in range(self.world):
            sx.state[r], sx.flags[r], sx.acks[r] = ent["state"].ptrs[r], ent["flags"].ptrs[r], ent["acks"].ptrs[r]
        sx.prefix, sx.words = ent["prefix"].data_ptr(), ent["words"].data_ptr()
        sx.wait_cycles, sx.rank, sx.world, sx.dir, sx.role = self.wait_cycles, self.rank, self.world, direction, role
        return ent["prefix"].view(bh, st)

    def _exchange(self, total: torch.Tensor, mode: int) -> torch.Tensor:
        if self.backend != "fused":
            parts = [torch.empty_like(total) for _ in range(self.world)]
            dist.all_gather(parts, total.contiguous(), group=self.group)
            take = [r for r in range(self.world) if mode == ALL or (mode == LOWER and r < self.rank) or (mode == HIGHER and r > self.rank)]
            out = torch.zeros_like(total)
            for r in take:
                out = out + parts[r]
            return out
        t = total.float().contiguous()
        n = t.numel()
        if n > self.max_numel or n % 4 != 0:
            raise ValueError(f"state of {n} elements does not fit this context ({self.max_numel}) or is not a multiple of 4")
        out = torch.empty_like(t)
        a = StateExchangeArgs()
        for r in range(self.world):
            a.slot[r], a.flags[r] = self.slot.ptrs[r], self.flags.ptrs[r]
        a.inp, a.out, a.numel = t.data_ptr(), out.data_ptr(), n
        a.rank, a.world, a.mode, a.epoch, a.wait_cycles = self.rank, self.world, mode, 0, self.wait_cycles
        a.words = self.words.data_ptr()
        a.status = nv.status_word(self.device).data_ptr()
        nv.check(nv.cuda().b200_state_exchange(C.byref(a), self.grid, nv.stream_ptr()), "state_exchange")
        nv.count_launch()
        self._keep = (t, out)
        return out.to(total.dtype).view(total.shape)

    def exclusive_prefix(self, total: torch.Tensor) -> torch.Tensor:
        return _ExchangeFn.apply(total, self, LOWER)

    def all_sum(self, total: torch.Tensor) -> torch.Tensor:
        return _ExchangeFn.apply(total, self, ALL)
