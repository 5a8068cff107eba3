"""Where the time of a training step goes (the reference's examples/profile_large.rs: forward only, forward + backward,
full step) for the 256-512-512-256 MLP at batch 64, plus the same step replayed as one CUDA graph and, with `--trace FILE`,
a `torch.profiler` Chrome trace with this package's NVTX ranges in it.

    python examples/profile_large.py [--trace step.json]
"""
import argparse
import time

import _common
import torch

from rust_neural_network_b200 import Adam, Linear, MSELoss, ReLU, Sequential, Trainer
from rust_neural_network_b200.utils import metrics

ap = argparse.ArgumentParser()
ap.add_argument("--trace", default="")
ap.add_argument("--iters", type=int, default=200)
args = ap.parse_args()
dev = _common.device()
torch.manual_seed(0)
model = Sequential().add(Linear(256, 512)).add(ReLU()).add(Linear(512, 512)).add(ReLU()).add(Linear(512, 256)).to_device(dev)
opt, loss_fn = Adam(model.parameters(), lr=1e-3), MSELoss("mean")
x, y = torch.randn(64, 256, device=dev), torch.randn(64, 256, device=dev)


def timed(fn):
    for _ in range(10):
        fn()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.iters):
        fn()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) / args.iters * 1e3


def fwd():
    with torch.no_grad():
        model(x)


def fwd_bwd():
    opt.zero_grad()
    loss_fn(model(x), y).backward()


def step():
    fwd_bwd()
    opt.step()


t_f, t_fb, t_s = timed(fwd), timed(fwd_bwd), timed(step)
print(f"forward            {t_f:8.4f} ms")
print(f"forward + backward {t_fb:8.4f} ms   (backward ~ {t_fb - t_f:.4f})")
print(f"full step          {t_s:8.4f} ms   (optimizer ~ {t_s - t_fb:.4f})")
if dev.type == "cuda":
    tr = Trainer(model, opt, loss_fn, use_cuda_graph=True)
    t_g = timed(lambda: tr.train_step(x, y))
    print(f"captured step      {t_g:8.4f} ms   ({tr.launches_per_step} kernels in one graph launch)")
    print(metrics.kernel_report())
if args.trace:
    with metrics.profile_to(args.trace):
        for _ in range(5):
            with metrics.nvtx_range("step"):
                step()
    print("trace written to", args.trace)
