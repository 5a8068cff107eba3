"""The ten benchmark groups of rust-nn benches/core_ops.rs (matmul, simd_matmul, attention, gemm_train, int8_vs_fp32,
blas_sgemm, dropout, fused_linear, elementwise, backward) at the reference's sizes, through this package's public API.

    python benches/core_ops.py                    # every group on the default device (cuda if present)
    python benches/core_ops.py attention dropout  # some groups
    python benches/core_ops.py --device cpu --quick

One line per case: group / case, median time, spread. On a GPU every case is timed with CUDA events after warm-up (the
median of `--iters` repetitions of a batch of `--batch` calls, so that a 5 us kernel is not timed through one event
pair); on CPU with `time.perf_counter`. These are latency numbers for small, launch-bound problems: the reference
measures them on one CPU core group, and the point of the table is which op costs what, not a roofline.
"""
from __future__ import annotations

import argparse
import math
import os
import statistics
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rust_neural_network_b200 import blas, int8, simd  # noqa: E402
from rust_neural_network_b200.fused import FusedActivation, fused_linear  # noqa: E402
from rust_neural_network_b200.linear_attention import KernelKind, linear_attention_forward  # noqa: E402
from rust_neural_network_b200.nn import Dropout, Linear, ReLU, Sequential  # noqa: E402
from rust_neural_network_b200.tensor import Tensor  # noqa: E402


class Bench:
    def __init__(self, device: str, iters: int, batch: int):
        self.dev, self.iters, self.batch = torch.device(device), iters, batch
        self.rows = []

    def t(self, *shape):
        return torch.randn(*shape, device=self.dev)

    def run(self, group: str, case: str, fn):
        for _ in range(3):
            fn()
        times = []
        if self.dev.type == "cuda":
            torch.cuda.synchronize()
            for _ in range(self.iters):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(self.batch):
                    fn()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) * 1e3 / self.batch)
        else:
            for _ in range(self.iters):
                t0 = time.perf_counter()
                for _ in range(self.batch):
                    fn()
                times.append((time.perf_counter() - t0) * 1e6 / self.batch)
        med, lo, hi = statistics.median(times), min(times), max(times)
        self.rows.append((group, case, med))
        print(f"{group + '/' + case:44s} {med:12.2f} us   [{lo:.2f} .. {hi:.2f}]", flush=True)


def bench_matmul(b: Bench, quick: bool):
    for size in ([64, 128] if quick else [64, 128, 256, 512]):
        x, y = Tensor(b.t(size, size)), Tensor(b.t(size, size))
        b.run("matmul", f"{size}x{size}", lambda: x.matmul(y))


def bench_simd_matmul(b: Bench, quick: bool):
    for size in ([64] if quick else [64, 128, 256]):
        i = torch.arange(size * size, dtype=torch.float32, device=b.dev)
        a, w, c = torch.sin(i * 0.001), torch.cos(i * 0.001), torch.zeros(size * size, device=b.dev)
        b.run("simd_matmul", f"{size}x{size}", lambda: simd.simd_matmul(a, w, c, size, size, size))


def bench_attention(b: Bench, quick: bool):
    batch, d = 2, 64
    scale = 1.0 / math.sqrt(d)
    for seq in ([128] if quick else [128, 512, 1024]):
        q, k, v = (Tensor(b.t(batch, seq, d)) for _ in range(3))
        b.run("attention", f"flash_seq{seq}", lambda: Tensor.flash_attention(q, k, v, scale))
        b.run("attention", f"linear_seq{seq}", lambda: linear_attention_forward(q.t, k.t, v.t, batch, seq, d, scale, 1e-6, False, KernelKind.Elu))


def bench_gemm_train(b: Bench, quick: bool):
    for label, m, n, k in (("fwd_b64", 64, 512, 512), ("fwd_b32", 32, 512, 512), ("dW_b64", 512, 512, 64)):
        a = torch.sin(torch.arange(m * k, dtype=torch.float32, device=b.dev) * 0.001)
        w = torch.cos(torch.arange(k * n, dtype=torch.float32, device=b.dev) * 0.001)
        c = torch.zeros(m * n, device=b.dev)
        b.run("gemm_train", label, lambda: blas.sgemm(blas.Transpose.NoTrans, blas.Transpose.NoTrans, m, n, k, 1.0, a, k, w, n, 0.0, c, n))


def bench_int8_vs_fp32(b: Bench, quick: bool):
    for n in ([256] if quick else [256, 512]):
        a, w, c = b.t(n * n), b.t(n * n), torch.zeros(n * n, device=b.dev)
        b.run("int8_vs_fp32", f"fp32_{n}", lambda: blas.sgemm(blas.Transpose.NoTrans, blas.Transpose.NoTrans, n, n, n, 1.0, a, n, w, n, 0.0, c, n))
        au = torch.randint(0, 128, (n * n,), dtype=torch.uint8, device=b.dev)
        bs = torch.randint(-128, 128, (n * n,), dtype=torch.int8, device=b.dev)
        b.run("int8_vs_fp32", f"int8_tensor_core_{n}", lambda: int8.igemm(au, bs, n, n, n))


def bench_blas_sgemm(b: Bench, quick: bool):
    for size in ([64, 128] if quick else [64, 128, 256, 512]):
        a, w, c = b.t(size * size), b.t(size * size), torch.zeros(size * size, device=b.dev)
        N, T = blas.Transpose.NoTrans, blas.Transpose.Trans
        b.run("blas_sgemm", f"blas_{size}x{size}", lambda: blas.sgemm(N, N, size, size, size, 1.0, a, size, w, size, 0.0, c, size))
        b.run("blas_sgemm", f"blas_transB_{size}x{size}", lambda: blas.sgemm(N, T, size, size, size, 1.0, a, size, w, size, 0.0, c, size))


def bench_dropout(b: Bench, quick: bool):
    for size in ([256] if quick else [256, 1024, 4096]):
        layer, x = Dropout(0.5), b.t(32, size)
        b.run("dropout", f"32x{size}", lambda: layer(x))


def bench_fused_linear(b: Bench, quick: bool):
    x, w, bias = b.t(32, 256), b.t(128, 256), b.t(128)
    b.run("fused_linear", "matmul+bias+relu", lambda: fused_linear(x, w, bias, FusedActivation.ReLU))
    layer = Linear(256, 128).to_device(b.dev) if b.dev.type == "cuda" else Linear(256, 128)
    relu = ReLU()
    b.run("fused_linear", "separate_matmul+bias+relu", lambda: relu(layer(x)))


def bench_elementwise(b: Bench, quick: bool):
    n = 65536
    x, y = b.t(n), b.t(n)
    out = torch.zeros(n, device=b.dev)
    b.run("elementwise", "simd_add_64k", lambda: simd.simd_add(x, y, out))
    b.run("elementwise", "simd_mul_64k", lambda: simd.simd_mul(x, y, out))
    b.run("elementwise", "simd_relu_64k", lambda: simd.simd_relu(x, out))
    b.run("elementwise", "simd_sum_64k", lambda: simd.simd_sum(x))


def bench_backward(b: Bench, quick: bool):
    model = Sequential().add(Linear(64, 128)).add(ReLU()).add(Linear(128, 64)).add(ReLU()).add(Linear(64, 10))
    if b.dev.type == "cuda":
        model.to_device(b.dev)
    x = b.t(8, 64)

    def step():
        for p in model.parameters():
            p.grad = None
        model(x).sum().backward()

    b.run("backward", "forward+backward", step)


GROUPS = {"matmul": bench_matmul, "simd_matmul": bench_simd_matmul, "attention": bench_attention, "gemm_train": bench_gemm_train,
          "int8_vs_fp32": bench_int8_vs_fp32, "blas_sgemm": bench_blas_sgemm, "dropout": bench_dropout, "fused_linear": bench_fused_linear,
          "elementwise": bench_elementwise, "backward": bench_backward}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("groups", nargs="*", help=f"any of: {' '.join(GROUPS)} (default: all)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=20, help="calls per timed repetition")
    ap.add_argument("--quick", action="store_true", help="the smallest size of every group only")
    args = ap.parse_args(argv)
    unknown = [g for g in args.groups if g not in GROUPS]
    if unknown:
        ap.error(f"unknown group(s): {unknown}")
    torch.manual_seed(0)
    b = Bench(args.device, args.iters, args.batch)
    for name in (args.groups or list(GROUPS)):
        GROUPS[name](b, args.quick)
    return 0


if __name__ == "__main__":
    sys.exit(main())
