"""Data parallelism (rust-nn src/distributed.rs, which only simulates it in-process).

`DistributedAdam` / `DistributedMuon` are the optimizers of a data-parallel job: one process per GPU,
identical initial weights, each rank computes gradients on its slice of the global batch, then the fused
kernels of csrc/comm/dp_fused.cu reduce-scatter the gradients over NVLink peer memory, apply the 1/world
scale, run the optimizer on the rank's slice of every bucket and all-gather the updated bf16 weights into
every rank's shadow buffer.

Layout of the flat parameter space (same on every rank):

* **sharded range** `[0, n_shard)`: the large matrices, which the forward only reads through their bf16
  shadow. It is cut into buckets at parameter boundaries; inside a bucket rank r owns the r-th of `world`
  equal slices. The fp32 master weights and optimizer state of a rank are authoritative only on the slices
  it owns (`prepare_checkpoint()` all-gathers them).
* **replicated range** `[n_shard, n)`: biases, norm gains and other small tensors, which the forward reads
  in fp32 (`is_replicated`). Every rank reduces these gradients from all peers in the same order and
  applies the same update, so their fp32 values are bit-identical everywhere.

Buckets overlap with backward when the model places `mark(h, k)` between its parameter groups and the
optimizer is given `groups=model.dp_groups()`: when backward passes the mark in front of group k, the
gradients of all groups >= k are final and their buckets are launched on a side stream.

Gradient clipping follows the reference (clip by the norm of the AVERAGED gradient, src/distributed.rs:507-523)
and Muon its per-tensor RMS rule (src/optim.rs:284-307); both need a norm of the reduced gradient, so they
run as two passes (reduce + sums of squares, then update) instead of one.

`mode="nccl"` is the baseline the fused path is measured against: NCCL all-reduce of the flat gradient
followed by the local optimizer kernel on every rank. On CPU ranks (gloo) the same class runs the
all-reduce path, which is what the host-logic tests use.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import kernels as K
from ..optim import FlatParams, Optimizer

DP_MAX_WORLD = 8
DP_MAX_CTAS = 160
REPLICATE_MAX_NUMEL = 1 << 18


class DpFusedArgs(C.Structure):
    _fields_ = [
        ("grad", C.c_void_p * DP_MAX_WORLD), ("shadow", C.c_void_p * DP_MAX_WORLD), ("flags", C.c_void_p * DP_MAX_WORLD),
        ("partial", C.c_void_p * DP_MAX_WORLD),
        ("grad_mc", C.c_void_p), ("shadow_mc", C.c_void_p),
        ("master", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
        ("begin", C.c_longlong), ("end", C.c_longlong), ("rep_begin", C.c_longlong), ("rep_end", C.c_longlong),
        ("rank", C.c_int), ("world", C.c_int),
        ("lr", C.c_float), ("b1", C.c_float), ("b2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float),
        ("torch_form", C.c_int), ("rule", C.c_int), ("scale_mode", C.c_int),
        ("step_ptr", C.c_void_p), ("grad_scale_ptr", C.c_void_p), ("words", C.c_void_p), ("status", C.c_void_p),
        ("wait_cycles", C.c_longlong),
        ("seg_off", C.c_void_p), ("blk_seg", C.c_void_p), ("nseg", C.c_int), ("first_rep_seg", C.c_int),
        ("red_rep", C.c_void_p), ("rep_sumsq", C.c_void_p), ("clip_max_norm", C.c_float), ("norm_out", C.c_void_p),
        ("bump_pass", C.c_int), ("red_scale", C.c_float),
    ]


nv.register_sigs({"b200_dp_fused_launch": [C.POINTER(DpFusedArgs), C.c_int, C.c_int, C.c_void_p], "b200_dp_flag_words": []})


def is_replicated(p: torch.Tensor, max_numel: int = REPLICATE_MAX_NUMEL) -> bool:
    """Parameters the forward reads in fp32 (biases, norm gains, conv taps, state matrices, routers) are kept
    identical on every rank instead of being sharded. `p._dp_replicate = True/False` overrides the size rule."""
    flag = getattr(p, "_dp_replicate", None)
    if flag is not None:
        return bool(flag)
    return p.dim() < 2 or p.numel() <= max_numel


GUARD_BYTES = 256
_GUARD_BYTE = 0xA5
_LIVE_BUFFERS: "weakref.WeakSet" = None


class SymmetricBuffer:
    """A tensor allocated in symmetric memory and mapped by every rank of the group.
    `ptrs[r]` is the address of rank r's copy in THIS process; `mc_ptr` is the NVLS multicast
    address (0 when unavailable).

    Every allocation carries a guard band of `GUARD_BYTES` on each side of the payload, filled with a fixed byte. The
    kernels that write through peer pointers are given the payload address only, so a store that runs past either end
    of a peer's buffer (a wrong shard offset, a row count that does not match) lands in a guard band instead of in a
    neighbouring allocation; `check()` / `check_canaries()` compare the bands with the pattern and name the buffer."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None, name: str = ""):
        import weakref

        import torch.distributed._symmetric_memory as symm_mem
        global _LIVE_BUFFERS
        group = group or dist.group.WORLD
        es = torch.empty((), dtype=dtype).element_size()
        g = GUARD_BYTES // es
        self.name = name or f"{dtype}[{numel}]"
        self._raw = symm_mem.empty(numel + 2 * g, dtype=dtype, device=device)
        self._raw.zero_()
        raw_bytes = self._raw.view(torch.uint8)
        raw_bytes[:GUARD_BYTES] = _GUARD_BYTE
        raw_bytes[GUARD_BYTES + numel * es:] = _GUARD_BYTE
        self.tensor = self._raw[g:g + numel]
        self.handle = symm_mem.rendezvous(self._raw, group)
        self.ptrs = [int(p) + GUARD_BYTES for p in self.handle.buffer_ptrs]
        mc = getattr(self.handle, "multicast_ptr", 0)
        self.mc_ptr = int(mc) + GUARD_BYTES if mc else 0
        if _LIVE_BUFFERS is None:
            _LIVE_BUFFERS = weakref.WeakSet()
        _LIVE_BUFFERS.add(self)

    def check(self) -> None:
        """Raise if anything (this rank or a peer) wrote outside the payload of this rank's copy."""
        b = self._raw.view(torch.uint8)
        n = self.tensor.numel() * self.tensor.element_size()
        front, back = b[:GUARD_BYTES], b[GUARD_BYTES + n:]
        bad_f, bad_b = int((front != _GUARD_BYTE).sum()), int((back != _GUARD_BYTE).sum())
        if bad_f or bad_b:
            raise RuntimeError(f"symmetric buffer {self.name}: {bad_f} bytes before and {bad_b} bytes after the payload were overwritten")


def check_canaries() -> int:
    """Check the guard bands of every live symmetric buffer of this process; returns how many were checked."""
    n = 0
    for buf in list(_LIVE_BUFFERS or ()):
        buf.check()
        n += 1
    return n


# ----------------------------------------------------------------------------------------------- marks
_ACTIVE: Optional["DistributedOptimizer"] = None


class _MarkFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, key):
        ctx.key = key
        return h.view_as(h)

    @staticmethod
    def backward(ctx, g):
        opt = _ACTIVE
        if opt is not None:
            opt.on_marker(ctx.key)
        return g, None


def mark(h: torch.Tensor, key: int) -> torch.Tensor:
    """Identity. Placed in a model's forward in FRONT of parameter group `key`: when backward passes it, the
    gradients of every group >= key are complete. Free when no bucketed data-parallel optimizer is active."""
    if _ACTIVE is None or not _ACTIVE.wants_marks or not h.requires_grad:
        return h
    return _MarkFn.apply(h, key)


class _Bucket:
    __slots__ = ("begin", "end", "first_group", "launched")

    def __init__(self, begin, end, first_group):
        self.begin, self.end, self.first_group, self.launched = begin, end, first_group, False


class DistributedOptimizer(Optimizer):
    """Shared machinery of the data-parallel optimizers. `rule` is "adam" or "muon". `average=False` SUMS the ranks'
    gradients instead of averaging them: the setting for the replicated parameters of a tensor / sequence parallel
    model, where every rank holds the gradient contribution of its own rows of one global batch."""

    def __init__(self, params, lr: float, rule: str, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 torch_compat: bool = False, momentum: float = 0.95, mode: str = "fused", group=None,
                 use_multimem: Optional[bool] = None, wait_seconds: float = 2.0, grid: int = 128,
                 groups: Optional[Sequence[Sequence[torch.Tensor]]] = None, bucket_mb: float = 32.0,
                 max_grad_norm: Optional[float] = None, overlap_grid: int = 32, average: bool = True,
                 replicate_max_numel: int = REPLICATE_MAX_NUMEL):
        global _ACTIVE
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        plist = [p for p in params if p.requires_grad]
        self.lr = float(lr)
        self.rule = rule
        dev = plist[0].device
        self.mode = mode if dev.type == "cuda" else "nccl"
        self.b1, self.b2 = (betas if rule == "adam" else (float(momentum), 0.0))
        self.eps, self.weight_decay, self.torch_compat = eps, weight_decay, torch_compat
        self.max_grad_norm = max_grad_norm
        self.red_scale = 1.0 / self.world if average else 1.0
        self.is_rep = lambda p: is_replicated(p, replicate_max_numel)
        is_rep = self.is_rep
        if rule == "muon" and max_grad_norm is not None:
            raise ValueError("Muon normalises every tensor's gradient by its RMS; clipping has no effect on it")

        # ---- layout: sharded parameters (in group order) first, replicated ones last
        if groups is not None:
            seen, ordered, group_of = set(), [], {}
            for gi, g in enumerate(groups):
                for p in g:
                    if p.requires_grad and id(p) not in seen:
                        seen.add(id(p)); ordered.append(p); group_of[id(p)] = gi
            rest = [p for p in plist if id(p) not in seen]
            for p in rest:                                      # parameters no group names: complete only after the whole backward
                group_of[id(p)] = -1
            ordered = rest + ordered
        else:
            ordered, group_of = list(plist), {id(p): -1 for p in plist}
        sharded = [p for p in ordered if not is_rep(p)]
        replicated = [p for p in ordered if is_rep(p)]
        self.params = plist
        self.flat = FlatParams(sharded + replicated, pad_to=64)
        fl = self.flat
        n = fl.numel
        first_rep = next((p for p in fl.order if is_rep(p)), None)
        self.n_shard = fl.offsets[id(first_rep)] if first_rep is not None else n
        assert self.n_shard % 64 == 0 and all((not is_rep(p)) == (fl.offsets[id(p)] < self.n_shard) for p in fl.order)
        self.n = n

        # ---- buckets: cut the sharded range at parameter boundaries (never inside a fused group)
        self.buckets: List[_Bucket] = []
        cur_begin, cur_group, prev_fuse = 0, None, None
        target = int(bucket_mb * (1 << 20) / 4)
        for p in fl.order:
            off = fl.offsets[id(p)]
            if off >= self.n_shard:
                break
            gi = group_of[id(p)]
            fuse = getattr(p, "_fuse_group", None)
            inside_fuse = fuse is not None and fuse is prev_fuse
            if cur_group is None:
                cur_group = gi
            elif gi != cur_group and not inside_fuse and off - cur_begin >= target and groups is not None:
                self.buckets.append(_Bucket(cur_begin, off, cur_group))
                cur_begin, cur_group = off, gi
            prev_fuse = fuse
        self.buckets.append(_Bucket(cur_begin, self.n_shard, cur_group if cur_group is not None else -1))
        self.wants_marks = self.mode == "fused" and len(self.buckets) > 1

        self.step_t = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_scale = None
        self._scalars = torch.zeros(4, dtype=torch.float32, device=dev)
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n if rule == "adam" else 1, dtype=torch.float32, device=dev)
        self.seg = fl.segments()
        self.grid = min(grid, DP_MAX_CTAS)
        self.overlap_grid = min(overlap_grid, self.grid)
        self._launched_in_backward = 0
        if self.mode == "fused":
            self._init_fused(dev, use_multimem, wait_seconds)
            _ACTIVE = self

    # ------------------------------------------------------------------ fused set-up
    def _init_fused(self, dev, use_multimem, wait_seconds):
        fl, n = self.flat, self.n
        if self.world > DP_MAX_WORLD:
            raise ValueError(f"fused data parallelism supports up to {DP_MAX_WORLD} ranks per group")
        # re-home gradient and shadow buffers into symmetric (peer-mapped) memory
        self.sym_grad = SymmetricBuffer(n, torch.float32, dev, self.group)
        self.sym_shadow = SymmetricBuffer(n, torch.bfloat16, dev, self.group)
        self.sym_flags = SymmetricBuffer(2 * DP_MAX_WORLD * DP_MAX_CTAS, torch.int32, dev, self.group)
        nseg = self.seg.shape[0]
        self.sym_partial = SymmetricBuffer(2 * max(nseg, 1), torch.float32, dev, self.group)
        with torch.no_grad():
            self.sym_shadow.tensor.copy_(fl.shadow)
        fl.grad = self.sym_grad.tensor
        fl.shadow = self.sym_shadow.tensor
        for p in fl.order:
            o, k = fl.offsets[id(p)], p.numel()
            p.grad = fl.grad[o:o + k].view(p.shape)
            p._lp = fl.shadow[o:o + k].view(p.shape)
            p._lp_version = p._version
            p._dp_sharded = o < self.n_shard and self.world > 1
        if use_multimem is None:
            use_multimem = os.environ.get("B200NN_DP_MULTIMEM", "0") == "1"
        self.use_multimem = bool(use_multimem and self.sym_grad.mc_ptr and self.sym_shadow.mc_ptr)
        # handshake epoch, retired-CTA counter, two-pass counter: device words that are NOT optimizer state
        self.words = torch.zeros(4, dtype=torch.int32, device=dev)
        starts = self.seg[:, 0].contiguous()
        blocks = torch.arange(0, (n + 1023) // 1024, device=dev, dtype=torch.int64) * 1024
        self.blk_seg = (torch.searchsorted(starts, blocks, right=True) - 1).clamp_min(0).to(torch.int32)
        self.first_rep_seg = int((starts < self.n_shard).sum().item())
        self.red_rep = torch.zeros(max(n - self.n_shard, 1), dtype=torch.float32, device=dev)
        self.rep_sumsq = torch.zeros(max(nseg, 1), dtype=torch.float32, device=dev)
        self.norm_out = self._scalars[2:3]
        a = DpFusedArgs()
        for r in range(self.world):
            a.grad[r], a.shadow[r], a.flags[r] = self.sym_grad.ptrs[r], self.sym_shadow.ptrs[r], self.sym_flags.ptrs[r]
            a.partial[r] = self.sym_partial.ptrs[r]
        a.grad_mc = self.sym_grad.mc_ptr if self.use_multimem else 0
        a.shadow_mc = self.sym_shadow.mc_ptr if self.use_multimem else 0
        a.master, a.m, a.v = fl.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr()
        a.rank, a.world = self.rank, self.world
        a.step_ptr, a.status, a.words = self.step_t.data_ptr(), nv.status_word(dev).data_ptr(), self.words.data_ptr()
        a.seg_off, a.blk_seg, a.nseg, a.first_rep_seg = self.seg.data_ptr(), self.blk_seg.data_ptr(), nseg, self.first_rep_seg
        a.red_rep, a.rep_sumsq, a.norm_out = self.red_rep.data_ptr(), self.rep_sumsq.data_ptr(), self.norm_out.data_ptr()
        a.rule = 0 if self.rule == "adam" else 1
        clock_hz = torch.cuda.get_device_properties(dev).clock_rate * 1000
        a.wait_cycles = int(wait_seconds * clock_hz)
        self._args = a
        self.comm_stream = torch.cuda.Stream(device=dev)
        dist.barrier(self.group)
        torch.cuda.synchronize()

    @property
    def two_pass(self) -> bool:
        return self.rule == "muon" or self.max_grad_norm is not None

    def _launch(self, pass_id: int, bucket: _Bucket, with_rep: bool, grid: int, bump: bool = False):
        a = DpFusedArgs.from_buffer_copy(self._args)
        a.lr, a.b1, a.b2, a.eps, a.weight_decay = self.lr, self.b1, self.b2, self.eps, self.weight_decay
        a.torch_form = int(self.torch_compat)
        a.grad_scale_ptr = nv.ptr(self.grad_scale)
        a.begin, a.end = bucket.begin, bucket.end
        a.rep_begin, a.rep_end = (self.n_shard, self.n) if with_rep else (self.n_shard, self.n_shard)
        a.scale_mode = 0 if pass_id == 0 else (2 if self.rule == "muon" else 1)
        a.clip_max_norm = float(self.max_grad_norm) if self.max_grad_norm is not None else 0.0
        a.bump_pass = int(bump)
        a.red_scale = self.red_scale
        nv.check(nv.cuda().b200_dp_fused_launch(C.byref(a), pass_id, grid, nv.stream_ptr()), "dp_fused_launch")
        nv.count_launch()

    # ------------------------------------------------------------------ overlap with backward
    def on_marker(self, key: int):
        """Backward has passed the mark in front of group `key`: reduce every bucket whose groups are all >= key."""
        if self.mode != "fused":
            return
        ready = [b for b in self.buckets if not b.launched and b.first_group >= key and b.first_group > 0]
        if not ready:
            return
        cur = torch.cuda.current_stream()
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            for b in sorted(ready, key=lambda b: -b.begin):
                self._launch(1 if self.two_pass else 0, b, False, self.overlap_grid)
                b.launched = True
                self._launched_in_backward += 1

    # ------------------------------------------------------------------ step
    def step(self):
        if self.mode == "fused":
            cur = torch.cuda.current_stream()
            if self._launched_in_backward:
                cur.wait_stream(self.comm_stream)
            rest = sorted([b for b in self.buckets if not b.launched], key=lambda b: -b.begin)
            for i, b in enumerate(rest):
                self._launch(1 if self.two_pass else 0, b, i == len(rest) - 1, self.grid)
            if self.two_pass:
                order = sorted(self.buckets, key=lambda b: b.begin)
                for i, b in enumerate(order):
                    last = i == len(order) - 1
                    self._launch(2, b, last, self.grid, bump=last)
            for b in self.buckets:
                b.launched = False
            self._launched_in_backward = 0
            nv.check(nv.cuda().b200_incr_step(self.step_t.data_ptr(), nv.stream_ptr()), "incr_step")
            nv.count_launch()
            return
        # baseline / CPU path: all-reduce the flat gradient, then the local optimizer kernel on every rank
        g = self.flat.grad
        if self.world > 1:
            dist.all_reduce(g, group=self.group)
        scale = torch.full((1,), self.red_scale, dtype=torch.float32, device=g.device)
        if self.grad_scale is not None:
            scale = scale * self.grad_scale
        if self.max_grad_norm is not None:
            # norm of the AVERAGED gradient (src/distributed.rs:507-523 clips after averaging)
            self._scalars.zero_()
            K.reduce_all(g, "sumsq", out=self._scalars[0:1])
            self._scalars[0:1].mul_(self.red_scale * self.red_scale)
            K.clip_coef(self._scalars, self.max_grad_norm)
            scale = scale * self._scalars[1:2]
        if self.rule == "adam":
            K.adam_step(self.flat.master, g, self.m, self.v, self.flat.shadow, self.lr, self.b1, self.b2,
                        self.eps, self.weight_decay, self.torch_compat, self.step_t, scale)
        else:
            g.mul_(scale)
            K.muon_rms_step(self.flat.master, g, self.m, self.flat.shadow, self.seg, self.lr, self.b1, self.eps)
            self.step_t.add_(1.0)

    def clip_grad_norm(self, max_norm: float):
        """Clip by the global norm of the gradient AVERAGED over the ranks, like the reference
        (src/distributed.rs:507-523). The norm only exists after the reduction, so this sets the threshold that
        `step()` applies; the returned 0-d device tensor holds the norm once `step()` has run."""
        if self.rule == "muon":
            raise ValueError("Muon normalises every tensor's gradient by its RMS; clipping has no effect on it")
        if self.max_grad_norm != max_norm:
            if self._launched_in_backward:
                raise RuntimeError("buckets of this step were already reduced during backward without clipping: "
                                   "pass max_grad_norm to the optimizer's constructor instead")
            self.max_grad_norm = float(max_norm)
        return self._scalars[2]

    # ------------------------------------------------------------------ checkpointing
    def _gather_full(self, t: torch.Tensor):
        for b in self.buckets:
            sh = (b.end - b.begin) // self.world
            if sh == 0:
                continue
            mine = t[b.begin + self.rank * sh: b.begin + (self.rank + 1) * sh].clone()
            dist.all_gather_into_tensor(t[b.begin:b.end], mine, group=self.group)

    def gather_master(self):
        """Make the fp32 master weights identical on all ranks (each rank is authoritative on the slices it owns)."""
        if self.mode != "fused" or self.world == 1:
            return
        self._gather_full(self.flat.master)

    def prepare_checkpoint(self):
        """Collective: all-gather the master weights and the optimizer moments so that `state_tensors()` and the
        model's parameters are complete on every rank and can be reloaded under any world size."""
        if self.mode != "fused" or self.world == 1:
            return
        self._gather_full(self.flat.master)
        self._gather_full(self.m)
        if self.rule == "adam":
            self._gather_full(self.v)

    def state_tensors(self):
        d = {"step": self.step_t, "m": self.m}
        if self.rule == "adam":
            d["v"] = self.v
        return d


class DistributedAdam(DistributedOptimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 torch_compat: bool = False, **kw):
        super().__init__(params, lr, "adam", betas=betas, eps=eps, weight_decay=weight_decay, torch_compat=torch_compat, **kw)


class DistributedMuon(DistributedOptimizer):
    """The reference's Muon (per-tensor RMS-normalised gradient, momentum SGD, src/optim.rs:284-307) under data
    parallelism: pass 1 reduces each rank's slice and accumulates per-tensor sums of squares, pass 2 combines the
    ranks' sums, updates the slice and all-gathers the bf16 weights."""

    def __init__(self, params, lr: float, momentum: float = 0.95, eps: float = 1e-8, **kw):
        super().__init__(params, lr, "muon", momentum=momentum, eps=eps, **kw)
