"""Training loop (rust-nn src/train.rs): `SimpleDataLoader` and `Trainer`.

`Trainer.train_epoch(loader)` = for each batch: zero_grad -> forward -> loss -> backward -> step,
returning the mean batch loss (src/train.rs:117-144). Batches are staged through pinned host
memory and copied to the model's device asynchronously; the per-batch losses stay on the device and
are read back once per epoch. `train_step` is the single-step entry point (host tensors in, loss
out) and can replay the whole step as one captured CUDA graph.
"""
from __future__ import annotations

from typing import Iterator, Optional, Tuple

import torch

from . import _native as nv


from ._compat import NewMixin as _NewMixin, unwrap as _unwrap  # noqa: E402

class SimpleDataLoader(_NewMixin):
    """Splits `inputs` / `targets` along dim 0 into batches of `batch_size`; no shuffle; the last
    batch may be short (src/train.rs:21-107)."""

    def __init__(self, inputs: torch.Tensor, targets: torch.Tensor, batch_size: int):
        from .tensor import Tensor as _W
        self._wrapped = isinstance(inputs, _W) or isinstance(targets, _W)      # built from wrappers: batches come out wrapped
        inputs = inputs.t if isinstance(inputs, _W) else inputs
        targets = targets.t if isinstance(targets, _W) else targets
        if inputs.shape[0] != targets.shape[0]:
            raise ValueError("inputs and targets must have the same number of rows")
        self.inputs, self.targets, self.batch_size = inputs, targets, max(1, int(batch_size))
        if torch.cuda.is_available() and not inputs.is_cuda:
            self.inputs = inputs.pin_memory()
            self.targets = targets.pin_memory()

    def __len__(self):
        return (self.inputs.shape[0] + self.batch_size - 1) // self.batch_size

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        n = self.inputs.shape[0]
        for i in range(0, n, self.batch_size):
            x, y = self.inputs[i:i + self.batch_size], self.targets[i:i + self.batch_size]
            if self._wrapped:
                from .tensor import Tensor as _W
                x, y = _W(x), _W(y)
            yield x, y

    __init__._accepts_wrapped = True           # unwraps by itself (it has to remember that it did)


class Trainer(_NewMixin):
    """`Trainer(model, optimizer, loss_fn)`; if `loss_fn` is None the model must expose
    `loss(inputs, targets)` (the fused LM head + cross-entropy path)."""

    def __init__(self, model, optimizer, loss_fn=None, use_cuda_graph: bool = False, grad_clip: Optional[float] = None,
                 logger=None, log_every: int = 1, tokens_per_step: int = 0):
        """`logger`: a `utils.metrics.MetricsLogger`; every `log_every` steps one record (step, loss, ms per step since the
        last record measured with CUDA events, tokens/s when `tokens_per_step` is given, kernel launches per step) is
        appended. Reading the loss for the record synchronises, so leave `logger` off in timed runs."""
        if isinstance(loss_fn, type):          # `Trainer::new(model, optimizer, MSELoss)`: a unit struct in the reference
            loss_fn = loss_fn()
        self.model, self.optimizer, self.loss_fn = model, optimizer, loss_fn
        self.logger, self.log_every, self.tokens_per_step = logger, max(1, int(log_every)), int(tokens_per_step)
        self._log_event = None
        self.use_cuda_graph = use_cuda_graph
        self.grad_clip = grad_clip
        if grad_clip is not None and hasattr(optimizer, "max_grad_norm"):
            optimizer.max_grad_norm = float(grad_clip)      # sharded optimizers clip inside their reduce passes
        self._graph = None
        self._static = None
        self.steps = 0

    # -- one optimisation step on device tensors
    def _step_device(self, x, y):
        from .utils.metrics import nvtx_range
        with nvtx_range("zero_grad"):
            self.optimizer.zero_grad()
        with nvtx_range("forward"):
            if self.loss_fn is None:
                loss = self.model.loss(x, y)
            else:
                loss = self.loss_fn(self.model(x), y)
        with nvtx_range("backward"):
            loss.backward()
        with nvtx_range("optimizer"):
            if self.grad_clip is not None:
                self.optimizer.clip_grad_norm(self.grad_clip)
            self.optimizer.step()
        return loss.detach()

    def _log(self, loss):
        if self.logger is None or self.steps % self.log_every:
            return
        rec = {"loss": float(loss)}
        if torch.cuda.is_available() and self.model.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            ev.synchronize()
            if self._log_event is not None:
                ms = self._log_event.elapsed_time(ev) / self.log_every
                rec["ms_per_step"] = ms
                if self.tokens_per_step:
                    rec["tokens_per_s"] = self.tokens_per_step / ms * 1e3
            self._log_event = ev
        if getattr(self, "launches_per_step", None):
            rec["launches_per_step"] = self.launches_per_step
        self.logger.log(self.steps, **rec)

    def _to_device(self, t, like_dtype=None):
        dev = self.model.device
        if t.device != dev:
            t = t.to(dev, non_blocking=True)
        if like_dtype is not None and t.is_floating_point() and t.dtype != like_dtype:
            t = t.to(like_dtype)
        return t

    def capture(self, x, y):
        """Capture zero_grad + forward + backward + optimizer step for inputs of this shape."""
        dev = self.model.device
        self._static = (torch.empty_like(x, device=dev), torch.empty_like(y, device=dev))
        self._static[0].copy_(x); self._static[1].copy_(y)
        # the warm-up steps below must not count as training: snapshot weights and optimizer state, restore after
        snap = []
        if hasattr(self.optimizer, "snapshot_tensors"):
            snap = [(t, t.clone()) for t in self.optimizer.snapshot_tensors()]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):                       # warm-up on a side stream (allocator, lazy init)
                self._step_device(*self._static)
            for t, saved in snap:
                t.copy_(saved)
        torch.cuda.current_stream().wait_stream(s)
        nv.check_status()
        self._graph = torch.cuda.CUDAGraph()
        before = nv.launch_count()
        with torch.cuda.graph(self._graph):
            self._static_loss = self._step_device(*self._static)
        self.launches_per_step = nv.launch_count() - before

    def train_step(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One step. Host tensors (ideally pinned) are copied to the device here. Returns the loss
        as a 0-d device tensor (call `.item()` / `float()` to read it back)."""
        cd = getattr(self.model, "compute_dtype", None)
        if self.use_cuda_graph and self.model.device.type == "cuda":
            if self._graph is None:
                self.capture(self._to_device(inputs, cd), self._to_device(targets))
            self._static[0].copy_(inputs, non_blocking=True)
            self._static[1].copy_(targets, non_blocking=True)
            self._graph.replay()
            self.steps += 1
            self._log(self._static_loss)
            return self._static_loss
        loss = self._step_device(self._to_device(inputs, cd), self._to_device(targets))
        self.steps += 1
        self._log(loss)
        return loss

    def train_epoch(self, loader) -> float:
        losses = []
        for x, y in loader:
            x, y = _unwrap(x), _unwrap(y)                          # a loader built from `Tensor` wrappers yields wrappers
            losses.append(self.train_step(x, y).clone())
        if not losses:
            return 0.0
        return float(torch.stack([l.float() for l in losses]).mean())


from ._compat import install as _install  # noqa: E402

_install(globals())
