"""Training steps per second of the four MLP shapes the reference publishes (its examples/bench_train.rs): a
d-h-h-out MLP with ReLU, sum-of-squares loss, Adam at 1e-2; five warm-up steps, then `steps` timed ones.

    python examples/bench_train.py [--graph]        # --graph: replay each step as one CUDA graph (GPU only)

`python bench_configs.py ref_mlp` prints the same shapes beside the reference's published numbers.
"""
import argparse
import time

import _common
import torch

from rust_neural_network_b200 import Adam, Linear, MSELoss, ReLU, Sequential, Trainer


def bench(d, h, out, batch, steps, label, dev, graph):
    torch.manual_seed(0)
    model = Sequential().add(Linear(d, h)).add(ReLU()).add(Linear(h, h)).add(ReLU()).add(Linear(h, out))
    model.to_device(dev)
    trainer = Trainer(model, Adam(model.parameters(), lr=1e-2), MSELoss(), use_cuda_graph=graph and dev.type == "cuda")
    x, y = torch.randn(batch, d, device=dev), torch.randn(batch, out, device=dev)
    for _ in range(5):
        trainer.train_step(x, y)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = trainer.train_step(x, y)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    print(f"{label}: d={d} h={h} out={out} batch={batch} steps={steps}  total={dt * 1e3:.2f}ms  per_step={dt / steps * 1e3:.3f}ms  loss={float(loss):.4f}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--scale", type=float, default=1.0, help="multiply the step counts (0.05 for a quick look)")
    a = ap.parse_args()
    dev = _common.device()
    for d, h, out, batch, steps, label in ((16, 32, 4, 8, 2000, "tiny"), (64, 128, 10, 32, 1000, "small"), (128, 256, 10, 32, 500, "medium"),
                                          (256, 512, 256, 64, 200, "large")):
        bench(d, h, out, batch, max(1, int(steps * a.scale)), label, dev, a.graph)
