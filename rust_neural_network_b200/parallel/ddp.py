"""Data parallelism (rust-nn src/distributed.rs, which only simulates it in-process).

`DistributedAdam` is the optimizer of a data-parallel job: one process per GPU, identical initial
weights, each rank computes gradients on its slice of the global batch, then ONE fused kernel per
step (csrc/comm/dp_fused.cu) reduce-scatters the gradients over NVLink peer memory, applies the
1/world scale (and clip coefficient), runs Adam on the rank's shard of the flat parameter space and
all-gathers the updated bf16 weights into every rank's shadow buffer. `mode="nccl"` is the baseline
the fused path is measured against: NCCL all-reduce of the flat gradient followed by the local Adam
kernel on every rank. On CPU ranks (gloo) the same class runs the all-reduce path, which is what the
host-logic tests use.

The fp32 master weights of a rank are authoritative only on its own shard; `gather_master()`
all-gathers them (checkpointing).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import kernels as K
from ..optim import Adam, FlatParams, Optimizer

DP_MAX_WORLD = 8
DP_MAX_CTAS = 160


class DpFusedArgs(C.Structure):
    _fields_ = [
        ("grad", C.c_void_p * DP_MAX_WORLD), ("shadow", C.c_void_p * DP_MAX_WORLD), ("flags", C.c_void_p * DP_MAX_WORLD),
        ("grad_mc", C.c_void_p), ("shadow_mc", C.c_void_p),
        ("master", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
        ("n", C.c_longlong), ("rank", C.c_int), ("world", C.c_int),
        ("lr", C.c_float), ("b1", C.c_float), ("b2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float),
        ("torch_form", C.c_int),
        ("step_ptr", C.c_void_p), ("grad_scale_ptr", C.c_void_p), ("status", C.c_void_p), ("wait_cycles", C.c_longlong),
    ]


nv.register_sigs({"b200_dp_fused_adam": [C.POINTER(DpFusedArgs), C.c_int, C.c_void_p], "b200_dp_flag_words": []})


class SymmetricBuffer:
    """A tensor allocated in symmetric memory and mapped by every rank of the group.
    `ptrs[r]` is the address of rank r's copy in THIS process; `mc_ptr` is the NVLS multicast
    address (0 when unavailable)."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        mc = getattr(self.handle, "multicast_ptr", 0)
        self.mc_ptr = int(mc) if mc else 0


class DistributedAdam(Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 torch_compat: bool = False, mode: str = "fused", group=None, use_multimem: Optional[bool] = None,
                 wait_seconds: float = 2.0, grid: int = 128):
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.params = [p for p in params if p.requires_grad]
        self.lr = float(lr)
        dev = self.params[0].device
        self.mode = mode if dev.type == "cuda" else "nccl"
        self.b1, self.b2 = betas
        self.eps, self.weight_decay, self.torch_compat = eps, weight_decay, torch_compat
        self.flat = FlatParams(self.params, pad_to=8 * self.world)
        n = self.flat.numel
        self.step_t = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_scale = None
        self._scalars = torch.zeros(4, dtype=torch.float32, device=dev)
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.grid = min(grid, DP_MAX_CTAS)
        if self.mode == "fused":
            # re-home gradient and shadow buffers into symmetric (peer-mapped) memory
            self.sym_grad = SymmetricBuffer(n, torch.float32, dev, self.group)
            self.sym_shadow = SymmetricBuffer(n, torch.bfloat16, dev, self.group)
            self.sym_flags = SymmetricBuffer(2 * DP_MAX_WORLD * DP_MAX_CTAS, torch.int32, dev, self.group)
            with torch.no_grad():
                self.sym_shadow.tensor.copy_(self.flat.shadow)
            self.flat.grad = self.sym_grad.tensor
            self.flat.shadow = self.sym_shadow.tensor
            for p in self.flat.order:
                o, k = self.flat.offsets[id(p)], p.numel()
                p.grad = self.flat.grad[o:o + k].view(p.shape)
                p._lp = self.flat.shadow[o:o + k].view(p.shape)
                p._lp_version = p._version
            if use_multimem is None:
                use_multimem = os.environ.get("B200NN_DP_MULTIMEM", "0") == "1"
            self.use_multimem = bool(use_multimem and self.sym_grad.mc_ptr and self.sym_shadow.mc_ptr)
            a = DpFusedArgs()
            for r in range(self.world):
                a.grad[r], a.shadow[r], a.flags[r] = self.sym_grad.ptrs[r], self.sym_shadow.ptrs[r], self.sym_flags.ptrs[r]
            a.grad_mc = self.sym_grad.mc_ptr if self.use_multimem else 0
            a.shadow_mc = self.sym_shadow.mc_ptr if self.use_multimem else 0
            a.master, a.m, a.v = self.flat.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr()
            a.n, a.rank, a.world = n, self.rank, self.world
            a.step_ptr, a.status = self.step_t.data_ptr(), nv.status_word(dev).data_ptr()
            clock_hz = torch.cuda.get_device_properties(dev).clock_rate * 1000
            a.wait_cycles = int(wait_seconds * clock_hz)
            self._args = a
            dist.barrier(self.group)
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ step
    def step(self):
        if self.mode == "fused":
            a = self._args
            a.lr, a.b1, a.b2, a.eps, a.weight_decay = self.lr, self.b1, self.b2, self.eps, self.weight_decay
            a.torch_form = int(self.torch_compat)
            a.grad_scale_ptr = nv.ptr(self.grad_scale)
            lib = nv.cuda()
            nv.check(lib.b200_dp_fused_adam(C.byref(a), self.grid, nv.stream_ptr()), "dp_fused_adam")
            nv.check(lib.b200_incr_step(self.step_t.data_ptr(), nv.stream_ptr()), "incr_step")
            nv.count_launch(2)
            return
        # baseline / CPU path: all-reduce the flat gradient, then the local fused Adam kernel
        dist.all_reduce(self.flat.grad, group=self.group)
        scale = torch.full((1,), 1.0 / self.world, dtype=torch.float32, device=self.flat.grad.device)
        if self.grad_scale is not None:
            scale = scale * self.grad_scale
        K.adam_step(self.flat.master, self.flat.grad, self.m, self.v, self.flat.shadow, self.lr, self.b1, self.b2,
                    self.eps, self.weight_decay, self.torch_compat, self.step_t, scale)

    def clip_grad_norm(self, max_norm: float):
        """Global norm over ALL ranks' averaged gradient is not available before the reduction; this
        clips by the norm of the local gradient averaged over ranks (an upper bound is not needed for
        the reference's semantics, src/distributed.rs:507-523, which clips after averaging)."""
        self._scalars.zero_()
        K.reduce_all(self.flat.grad, "sumsq", out=self._scalars[0:1])
        if self.world > 1:
            dist.all_reduce(self._scalars[0:1], group=self.group)
            self._scalars[0:1].div_(self.world)
        K.clip_coef(self._scalars, max_norm)
        self.grad_scale = self._scalars[1:2]
        return self._scalars[2]

    def gather_master(self):
        """Make the fp32 master weights identical on all ranks (each rank is authoritative on its shard)."""
        if self.mode != "fused" or self.world == 1:
            return
        shard = self.flat.numel // self.world
        parts = [self.flat.master[r * shard:(r + 1) * shard] for r in range(self.world)]
        dist.all_gather(parts, parts[self.rank].clone(), group=self.group)

    def state_tensors(self):
        return {"step": self.step_t, "m": self.m, "v": self.v}
