"""`CompiledMLP` on the reference's "large" shape (its examples/bench_compiled.rs): 256-512-512-256, batch 64, lr 0.01,
deterministic sin / cos data, five warm-up steps, 500 timed.

    python examples/bench_compiled.py [--iters N]
"""
import argparse
import time

import _common
import torch

from rust_neural_network_b200.compiled import CompiledMLP

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=500)
    a = ap.parse_args()
    dev = _common.device()
    m = CompiledMLP.new([(256, 512), (512, 512), (512, 256)], 64, 0.01)
    i = torch.arange(64 * 256, dtype=torch.float32)
    x, t = torch.sin(i * 0.001).reshape(64, 256), torch.cos(i * 0.001).reshape(64, 256)
    for _ in range(5):
        m.step(x, t)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.iters):
        loss = m.step(x, t)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / a.iters * 1e3
    print(f"compiled large (256-512-512-256, b64): {dt:.3f} ms/step  loss {float(loss):.5f}")
