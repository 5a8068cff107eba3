"""GEMM throughput and a checksum over the shapes a Linear layer produces (the reference's examples/gemm_shapes.rs):
forward x W^T, input gradient dY W, weight gradient dY^T x. On a GPU this is the tcgen05 kernel timed with CUDA events;
on a CPU-only machine it times the C++ restatement of the reference's packed AVX2 sgemm.

    python examples/gemm_shapes.py
"""
import time

import _common
import torch

from rust_neural_network_b200 import cpu_ref
from rust_neural_network_b200.ops.gemm import gemm

dev = _common.device()
shapes = [(64, 512, 256), (64, 512, 512), (64, 256, 512), (512, 512, 512), (4096, 2048, 512), (8192, 8192, 2048)]
print(f"{'M':>6} {'N':>6} {'K':>6} {'layout':>8} {'ms':>9} {'GFLOP/s':>10}  checksum")
for m, n, k in shapes:
    if dev.type == "cpu" and m * n * k > 512 ** 3:
        continue
    g = torch.Generator().manual_seed(m + n + k)
    a, b = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
    for layout in ("NT", "NN", "TN"):
        if dev.type == "cuda":
            A = (a if layout != "TN" else a.t().contiguous()).to(dev, torch.bfloat16)
            B = (b if layout == "NT" else b.t().contiguous()).to(dev, torch.bfloat16)
            run = lambda: gemm(A, B, a_mn=layout == "TN", b_mn=layout != "NT")
            out = run()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                out = run()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 20
        else:
            A = a if layout != "TN" else a.t().contiguous()
            B = b if layout == "NT" else b.t().contiguous()
            run = lambda: cpu_ref.sgemm(A, B, trans_a=layout == "TN", trans_b=layout == "NT", threads=1)
            out = run()
            t0 = time.perf_counter()
            for _ in range(5):
                out = run()
            ms = (time.perf_counter() - t0) / 5 * 1e3
        print(f"{m:6d} {n:6d} {k:6d} {layout:>8} {ms:9.4f} {2.0 * m * n * k / ms / 1e6:10.1f}  {float(out.float().sum()):.3f}")
