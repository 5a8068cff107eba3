"""Single-kernel micro-benchmarks with roofline fractions.

    python -m rust_neural_network_b200.utils.kernel_bench gemm --m 65536 --n 2048 --k 512 [--bias --act gelu --residual]
    python -m rust_neural_network_b200.utils.kernel_bench gemm_mx --m 8192 --n 8192 --k 8192 --kind mxfp8|nvfp4
    python -m rust_neural_network_b200.utils.kernel_bench flash_fwd --b 64 --s 1024 --h 8 --hd 64 --causal
    python -m rust_neural_network_b200.utils.kernel_bench flash_bwd ...
    python -m rust_neural_network_b200.utils.kernel_bench layernorm_bwd --rows 65536 --d 512
    python -m rust_neural_network_b200.utils.kernel_bench scan_fwd --b 8 --s 4096 --d 4096 --n 16

Timing: CUDA events on the launching stream, >= 3 warm-up iterations, an L2 flush (a write of a
buffer larger than L2) before every timed iteration, median over the timed iterations. The
denominators come from MEASURED_PEAKS.json at the repository root when present ("of measured"),
otherwise the fallback figures 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "of measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "of fallback"}


class L2Flusher:
    def __init__(self, dev):
        self.buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.zero_()


def time_fn(fn, iters=10, warmup=3):
    """Median device time of `fn` in ms. Each timed call follows an L2 flush; the sequence (flush, fn) x iters is
    recorded into a CUDA graph and replayed, and a second graph with the flushes alone is subtracted, so neither
    host launch latency nor the flush itself is in the number."""
    dev = torch.device("cuda")
    flush = L2Flusher(dev)
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()

    def capture(with_fn):
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            flush()
            if with_fn:
                fn()
        torch.cuda.current_stream().wait_stream(s)
        with torch.cuda.graph(g):
            for _ in range(iters):
                flush()
                if with_fn:
                    fn()
        return g

    def replay_ms(g):
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); g.replay(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]

    g_both, g_flush = capture(True), capture(False)
    replay_ms(g_both); replay_ms(g_flush)
    return max(replay_ms(g_both) - replay_ms(g_flush), 0.0) / iters


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_mx", "flash_fwd", "flash_bwd", "layernorm_bwd", "layernorm_fwd", "ce", "scan_fwd", "scan_bwd"])
    for name, default in (("m", 65536), ("n", 2048), ("k", 512), ("b", 64), ("s", 1024), ("h", 8), ("hd", 64),
                          ("rows", 65536), ("d", 512), ("v", 32000), ("iters", 10)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--act", default="none")
    ap.add_argument("--dact", default="none", help="multiply the GEMM result by act'(saved pre-activation) in the epilogue (fused activation backward)")
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--f32-out", action="store_true")
    ap.add_argument("--kind", default="mxfp8", choices=["mxfp8", "nvfp4"], help="gemm_mx: block-scaled operand format")
    ap.add_argument("--bn", type=int, default=0, help="GEMM tile width override (64 / 128 / 256)")
    args = ap.parse_args(argv)

    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops import gemm as G
    from rust_neural_network_b200.ops import kernels as K
    nv.cuda()
    dev = "cuda"
    pk = peaks()
    out = {"kernel": args.kernel, "peaks": pk}
    torch.manual_seed(0)

    if args.kernel == "gemm":
        M, N, Kd = args.m, args.n, args.k
        a = torch.randn((Kd, M) if args.a_mn else (M, Kd), device=dev).bfloat16()
        b = torch.randn((Kd, N) if args.b_mn else (N, Kd), device=dev).bfloat16()
        bias = torch.randn(N, device=dev) if args.bias else None
        res = torch.randn(M, N, device=dev).bfloat16() if args.residual else None
        aux_in = torch.randn(M, N, device=dev).bfloat16() if args.dact != "none" else None
        kw = dict(a_mn=args.a_mn, b_mn=args.b_mn, bias=bias, act=args.act, residual=res, want_aux=args.act in ("gelu", "silu"),
                  out_dtype=torch.float32 if args.f32_out else None, bn=args.bn, aux_in=aux_in, dact=args.dact)
        ms = time_fn(lambda: G.gemm(a, b, **kw), args.iters)
        flops = 2.0 * M * N * Kd
        byts = 2.0 * (M * Kd + N * Kd) + (4.0 if args.f32_out else 2.0) * M * N * (2 if kw["want_aux"] else 1) + (2.0 * M * N if res is not None else 0) + (2.0 * M * N if aux_in is not None else 0)
        out.update(shape=[M, N, Kd], ms=ms, tflops=flops / ms / 1e9, frac_of_bf16_peak=flops / ms / 1e9 / pk["bf16_tflops"],
                   gbs=byts / ms / 1e6, frac_of_hbm_peak=byts / ms / 1e6 / pk["hbm_gbs"])
    elif args.kernel == "gemm_mx":
        from rust_neural_network_b200.ops import mx
        M, N, Kd = args.m, args.n, args.k
        qa = mx.quantize_mx(torch.randn(M, Kd, device=dev).bfloat16(), args.kind)
        qb = mx.quantize_mx(torch.randn(N, Kd, device=dev).bfloat16(), args.kind)
        ms = time_fn(lambda: mx.gemm_mx(qa, qb), args.iters)
        xq = torch.randn(M, Kd, device=dev).bfloat16()
        ms_q = time_fn(lambda: mx.quantize_mx(xq, args.kind, tensor_scale=qa.tensor_scale), args.iters)      # scale given: no host sync
        flops = 2.0 * M * N * Kd
        out.update(shape=[M, N, Kd], kind=args.kind, ms=ms, tflops=flops / ms / 1e9, vs_bf16_peak=flops / ms / 1e9 / pk["bf16_tflops"],
                   quantise_activations_ms=ms_q, nominal_dense_peak_tflops=4500.0 if args.kind == "mxfp8" else 9000.0)
    elif args.kernel in ("flash_fwd", "flash_bwd"):
        B, S, H, hd = args.b, args.s, args.h, args.hd
        qkv = (torch.randn(B, S, 3, H, hd, device=dev) * 0.5).bfloat16()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        scale = 1.0 / math.sqrt(hd)
        o, lse = K.flash_fwd(q, k, v, scale, args.causal)
        flops = 4.0 * B * H * S * S * hd * (0.5 if args.causal else 1.0)
        if args.kernel == "flash_fwd":
            ms = time_fn(lambda: K.flash_fwd(q, k, v, scale, args.causal), args.iters)
        else:
            do = torch.randn_like(o)
            dqkv = torch.empty_like(qkv)
            ms = time_fn(lambda: K.flash_bwd(do, q, k, v, o, lse, scale, args.causal, dq=dqkv[:, :, 0], dk=dqkv[:, :, 1], dv=dqkv[:, :, 2]), args.iters)
            flops *= 2.5
        out.update(shape=[B, S, H, hd], causal=args.causal, ms=ms, tflops=flops / ms / 1e9, frac_of_bf16_peak=flops / ms / 1e9 / pk["bf16_tflops"])
    elif args.kernel in ("layernorm_bwd", "layernorm_fwd"):
        rows, d = args.rows, args.d
        x = torch.randn(rows, d, device=dev).bfloat16(); dy = torch.randn_like(x)
        g = torch.ones(d, device=dev); bta = torch.zeros(d, device=dev)
        y, mean, rstd = K.layernorm_fwd(x, g, bta, 1e-5)
        if args.kernel == "layernorm_fwd":
            ms = time_fn(lambda: K.layernorm_fwd(x, g, bta, 1e-5), args.iters); byts = 2.0 * rows * d * 2
        else:
            ms = time_fn(lambda: K.layernorm_bwd(dy, x, g, mean, rstd, dres=dy), args.iters); byts = 2.0 * rows * d * 4
        out.update(shape=[rows, d], ms=ms, gbs=byts / ms / 1e6, frac_of_hbm_peak=byts / ms / 1e6 / pk["hbm_gbs"])
    elif args.kernel == "ce":
        rows, V = args.rows, args.v
        logits = torch.randn(rows, V, device=dev).bfloat16(); labels = torch.randint(0, V, (rows,), device=dev)
        ms = time_fn(lambda: K.ce_label(logits, labels), args.iters)
        byts = 2.0 * rows * V * 2
        out.update(shape=[rows, V], ms=ms, gbs=byts / ms / 1e6, frac_of_hbm_peak=byts / ms / 1e6 / pk["hbm_gbs"])
    else:
        from rust_neural_network_b200.ops import scan as SC
        B, S, D, N = args.b, args.s, args.d, args.n if args.n <= 16 else 16
        u = torch.randn(B, S, D, device=dev).bfloat16(); delta = (torch.randn(B, S, D, device=dev) * 0.5).bfloat16()
        A = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).repeat(D, 1)
        Bm = torch.randn(B, S, N, device=dev).bfloat16(); Cm = torch.randn(B, S, N, device=dev).bfloat16()
        z = torch.randn(B, S, D, device=dev).bfloat16()
        # as the Mamba block runs it: the gate y * silu(z) is its own elementwise kernel beside the 16-state lane kernels
        from rust_neural_network_b200.ops import kernels as K
        gate_outside = N == 16
        zk = None if gate_outside else z
        y, hck = SC.scan_fwd_raw(u, delta, A, Bm, Cm, None, zk, None, True, True)
        byts = 2.0 * B * S * D * 4
        if args.kernel == "scan_fwd":
            def fwd():
                yy, _ = SC.scan_fwd_raw(u, delta, A, Bm, Cm, None, zk, None, True, True)
                return K.binary(yy, z, "mul_silu") if gate_outside else yy
            ms = time_fn(fwd, args.iters)
        else:
            dy = torch.randn_like(y)
            def bwd():
                g = K.binary(dy, z, "mul_silu") if gate_outside else dy
                return SC.scan_bwd_raw(g, u, delta, A, Bm, Cm, None, zk, None, True, hck)
            ms = time_fn(bwd, args.iters)
            byts *= 2
        out.update(shape=[B, S, D, N], ms=ms, gbs=byts / ms / 1e6, frac_of_hbm_peak=byts / ms / 1e6 / pk["hbm_gbs"],
                   exps_per_s=B * S * D * N / ms * 1e3)
    nv.check_status()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
