"""Benchmarks of the configurations beside the headline one (which `bench.py` measures).

    python bench_configs.py mlp                     784-256-128-10 MLP, fp32/TF32, batch 32, Adam, CUDA-graph step
    python bench_configs.py ref_mlp                 the four MLP shapes the reference publishes step times for: GPU graph step,
                                                    C++ restatement of the reference's CPU path, published numbers
    python bench_configs.py moe_lm   [--batch B]    FineGrainedMoE transformer LM (64 routed top-6 + 2 shared)
    python bench_configs.py mamba_lm [--batch B]    Mamba (S6) LM, d 2048, 24 layers, seq 4096
    python -m torch.distributed.run --nproc-per-node N ... bench_configs.py moe_lm      expert parallel, 64/N experts per GPU
    python -m torch.distributed.run --nproc-per-node N ... bench_configs.py mamba_lm    N-way tensor parallel
        add --impl torch for the NCCL + cuBLAS library arm of either, --comm nccl for this package's kernels with NCCL
        calls instead of the fused communication kernels
    python bench_configs.py attention --seq 4096 --head-dim 64      forward+backward: flash vs causal linear attention
    python -m torch.distributed.run --nproc-per-node 8 ... bench_configs.py attention_sp --seq 65536
                                                    sequence-parallel causal linear attention (KV-state exchange kernel)

Every run prints one JSON line. Steps are timed on the device with CUDA events after >= 3 warm-up steps; the
training configurations move hundreds of MB to GB per step, far above the 126 MB L2; the attention sweep flushes
L2 between iterations. One GPU per process; launch the LM configurations under torch.distributed.run for
data-parallel runs (`DistributedAdam` picks the fused reduce-scatter + Adam kernel).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

import torch


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _setup_dist():
    import torch.distributed as dist
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, dev


def _time_steps(step, args, world, dev):
    """>= 3 warm-up steps, then `args.steps` steps between CUDA events; max over ranks. Returns (ms, first loss, last loss)."""
    import torch.distributed as dist
    first = None
    for i in range(max(args.warmup, 3)):
        l = step(i)
        first = float(l) if first is None else first
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = _events()
    e0.record()
    last = 0.0
    for i in range(args.steps):
        last = float(step(i).item())
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, first, last


def _kernel_table(step, path, rank):
    """One more step under `torch.profiler` (after the timed region; never a timed number): device time per kernel name,
    largest first, written by rank 0. Shares of the step, for deciding which kernel to look at next."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    if rank != 0:
        return
    rows = {}
    for ka in prof.key_averages():
        t = getattr(ka, "self_device_time_total", 0) or 0
        if t:
            rows[ka.key] = (float(t), int(ka.count))
    total = sum(v[0] for v in rows.values()) or 1.0
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write(f"# device time by kernel over one step, total {total / 1e3:.2f} ms (profiler run: shares, not a timing)\n")
        for name, (t, c) in sorted(rows.items(), key=lambda kv: -kv[1][0])[:60]:
            f.write(f"{100 * t / total:6.2f} %  {t / 1e3:9.3f} ms  x{c:<5d} {name[:150]}\n")


def run_lm(name, args):
    """b200 arm: this package's kernels. `--parallel` picks the layout for N > 1: `tp` (Mamba: channel-sharded blocks on
    row-sharded activations, fused all-gather->GEMM / GEMM->reduce-scatter / all-reduce kernels), `ep` (MoE: experts
    sharded over the ranks, peer-memory dispatch / combine, data-parallel shared parameters), `dp` (plain data parallel).
    `--comm nccl` keeps the package's kernels but replaces the fused communication kernels by NCCL calls."""
    import torch.distributed as dist
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.config import PRESETS, build_model
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.train import Trainer

    world, rank, dev = _setup_dist()
    over = {}
    if args.layers:
        over["layers"] = args.layers
    if args.seq:
        over["seq_len"] = args.seq
    if args.recompute_scan and name == "mamba_lm":
        over["recompute_scan"] = True
    cfg = dataclasses.replace(PRESETS[name], **over)
    batch = args.batch or getattr(cfg, "batch_per_gpu", 0) or cfg.global_batch // world
    par = args.parallel if args.parallel != "auto" else (cfg.parallelism if world > 1 else "none")
    if world == 1:
        par = "none"
    torch.manual_seed(1234)
    extra = {}
    if par == "tp":
        from rust_neural_network_b200.parallel.tp import TPContext
        M = world * batch * cfg.seq_len
        extra["tp"] = TPContext(M, cfg.d_model, cfg.d_model, device=dev, backend="fused" if args.comm == "fused" else "nccl",
                                max_allreduce_numel=M * (cfg.dt_rank + 2 * cfg.d_state))
    elif par == "ep":
        extra["ep_group"] = dist.group.WORLD
        extra["ep_backend"] = args.comm
    model, cfg = build_model(name, dev, **over, **extra)
    if par in ("tp", "ep"):
        opt = model.make_optimizer(lr=1e-3) if par == "tp" else model.make_optimizer(lr=1e-3, mode=args.comm)
    elif world > 1:
        from rust_neural_network_b200.parallel.ddp import DistributedAdam
        groups = model.dp_groups() if (args.buckets and hasattr(model, "dp_groups")) else None
        opt = DistributedAdam(model.parameters(), lr=1e-3, mode=args.comm, groups=groups)
    else:
        opt = Adam(model.parameters(), lr=1e-3)
    graph = not args.no_graph and not (par == "ep" and args.comm == "nccl")     # host-side split sizes cannot be captured
    tr = Trainer(model, opt, loss_fn=None, use_cuda_graph=graph)
    g = torch.Generator().manual_seed(1000 + rank)
    ids = [torch.randint(0, cfg.vocab, (batch, cfg.seq_len), generator=g).pin_memory() for _ in range(2)]
    lab = [torch.randint(0, cfg.vocab, (batch, cfg.seq_len), generator=g).pin_memory() for _ in range(2)]
    ms, first, last = _time_steps(lambda i: tr.train_step(ids[i % 2], lab[i % 2]), args, world, dev)
    nv.check_status()
    if args.kernel_table:
        _kernel_table(lambda: tr.train_step(ids[0], lab[0]), args.kernel_table, rank)
    n_params = sum(p.numel() for p in model.parameters())
    if rank == 0:
        print(json.dumps({"config": name, "impl": "b200", "comm": args.comm, "parallel": par, "n_gpus": world, "batch_per_gpu": batch,
                          "seq_len": cfg.seq_len, "preset": dataclasses.asdict(cfg), "params_per_rank": n_params, "ms_per_step": ms,
                          "tokens_per_s": world * batch * cfg.seq_len / ms * 1e3, "end_to_end": True, "cuda_graph": tr._graph is not None,
                          "launches_per_step": getattr(tr, "launches_per_step", None), "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
                          "loss_first": first, "loss_last": last}), flush=True)
    if world > 1:
        tr._graph = None
        sys.stdout.flush()
        os._exit(0)


def run_lm_torch(name, args):
    """Library arm of the MoE / Mamba configurations (baseline/torch_moe.py, baseline/torch_mamba.py): NCCL collectives
    around cuBLAS GEMMs, stock PyTorch everywhere it has the op. Same shapes, precision policy and timing rules."""
    import torch.distributed as dist
    from rust_neural_network_b200.config import PRESETS

    world, rank, dev = _setup_dist()
    over = {}
    if args.layers:
        over["layers"] = args.layers
    if args.seq:
        over["seq_len"] = args.seq
    cfg = dataclasses.replace(PRESETS[name], **over)
    batch = args.batch or cfg.batch_per_gpu
    torch.manual_seed(1234)
    group = dist.group.WORLD if world > 1 else None
    if name == "moe_lm":
        from baseline.torch_moe import TorchMoELM, TorchMoEStep
        model = TorchMoELM(cfg.vocab, cfg.d_model, cfg.layers, cfg.heads, cfg.num_experts, cfg.top_k, cfg.num_shared, cfg.expert_hidden,
                           cfg.seq_len, world, rank, group).to(dev)
        stepper = TorchMoEStep(model, world, group)
        par = "ep" if world > 1 else "none"
    else:
        from baseline.torch_mamba import TorchMambaLM, TorchMambaStep
        model = TorchMambaLM(cfg.vocab, cfg.d_model, cfg.layers, cfg.d_state, cfg.d_conv, cfg.expand, cfg.dt_rank, world, rank, group).to(dev)
        stepper = TorchMambaStep(model, world, group)
        par = "tp" if world > 1 else "none"
    g = torch.Generator().manual_seed(1000 + rank)
    ids = [torch.randint(0, cfg.vocab, (batch, cfg.seq_len), generator=g).pin_memory() for _ in range(2)]
    lab = [torch.randint(0, cfg.vocab, (batch, cfg.seq_len), generator=g).pin_memory() for _ in range(2)]
    ms, first, last = _time_steps(lambda i: stepper.step(ids[i % 2].to(dev, non_blocking=True), lab[i % 2].to(dev, non_blocking=True)), args, world, dev)
    if args.kernel_table:
        _kernel_table(lambda: stepper.step(ids[0].to(dev, non_blocking=True), lab[0].to(dev, non_blocking=True)), args.kernel_table, rank)
    if rank == 0:
        print(json.dumps({"config": name, "impl": "torch", "comm": "nccl", "parallel": par, "n_gpus": world, "batch_per_gpu": batch,
                          "seq_len": cfg.seq_len, "params_per_rank": sum(p.numel() for p in model.parameters()), "ms_per_step": ms,
                          "tokens_per_s": world * batch * cfg.seq_len / ms * 1e3, "end_to_end": True, "cuda_graph": False,
                          "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30, "loss_first": first, "loss_last": last}), flush=True)
    if world > 1:
        sys.stdout.flush()
        os._exit(0)


def run_mlp(args):
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200 import loss as L
    from rust_neural_network_b200.config import build_model
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.train import Trainer

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    model, cfg = build_model("mlp", dev)
    tr = Trainer(model, Adam(model.parameters(), lr=cfg.lr), L.CrossEntropyLoss(), use_cuda_graph=not args.no_graph)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(cfg.batch, cfg.dims[0], generator=g).pin_memory()
    y = torch.nn.functional.one_hot(torch.randint(0, cfg.dims[-1], (cfg.batch,), generator=g), cfg.dims[-1]).float().pin_memory()
    first = float(tr.train_step(x, y))
    for _ in range(4):
        tr.train_step(x, y)
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    for _ in range(cfg.steps):
        l = tr.train_step(x, y)
    e1.record()
    torch.cuda.synchronize()
    nv.check_status()
    ms = e0.elapsed_time(e1) / cfg.steps
    print(json.dumps({"config": "mlp", "impl": "b200", "dims": list(cfg.dims), "batch": cfg.batch, "dtype": "fp32 storage, TF32 tensor-core products",
                      "us_per_step": ms * 1e3, "samples_per_s": cfg.batch / ms * 1e3, "steps": cfg.steps, "cuda_graph": tr._graph is not None,
                      "launches_per_step": getattr(tr, "launches_per_step", None), "loss_first": first, "loss_last": float(l)}), flush=True)


# MLP shapes the reference publishes step times for (its README: rust-nn autograd / CompiledMLP against PyTorch eager,
# single CPU thread, Adam + MSE; examples/bench_train.rs:44-47, examples/bench_compiled.rs)
REF_MLP_SHAPES = [
    ("tiny", (16, 32, 32, 4), 8, {"rust_nn_ms": 0.032, "pytorch_cpu_ms": 0.770}),
    ("small", (64, 128, 128, 10), 32, {"rust_nn_ms": 0.35, "pytorch_cpu_ms": 0.82}),
    ("medium", (128, 256, 256, 10), 32, {"rust_nn_ms": 1.2, "pytorch_cpu_ms": 1.25}),
    ("large", (256, 512, 512, 256), 64, {"rust_nn_ms": 6.5, "rust_nn_compiled_ms": 4.68, "rust_nn_compiled_2thread_ms": 3.95, "pytorch_cpu_ms": 4.1}),
]


def run_ref_mlp(args):
    """The four published MLP shapes, three ways: this package on the GPU (`CompiledMLP`: the whole step replayed as one
    CUDA graph, inputs copied from pinned host memory every step), the C++ restatement of the reference's CPU path
    (`cpu_ref.CpuMLP`, packed AVX2 sgemm + AVX2 Adam, 1 and 2 threads) on this machine's CPU, and the published numbers."""
    import time
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200 import cpu_ref
    from rust_neural_network_b200.compiled import CompiledMLP
    rows = []
    steps = max(args.steps, 200)
    for name, dims, batch, pub in REF_MLP_SHAPES:
        g = torch.Generator().manual_seed(0)
        x, y = torch.randn(batch, dims[0], generator=g), torch.randn(batch, dims[-1], generator=g)
        rec = {"shape": name, "dims": list(dims), "batch": batch, "published": pub}
        for th in (1, 2):
            net = cpu_ref.CpuMLP(dims, seed=0)
            for _ in range(20):
                net.step(x, targets=y, threads=th)
            t0 = time.perf_counter()
            for _ in range(steps):
                net.step(x, targets=y, threads=th)
            rec[f"cpu_restatement_{th}thread_ms"] = (time.perf_counter() - t0) / steps * 1e3
        if torch.cuda.is_available():
            m = CompiledMLP([(dims[i], dims[i + 1]) for i in range(len(dims) - 1)], batch, 1e-3)
            xp, yp = x.pin_memory(), y.pin_memory()
            first = m.step(xp, yp)
            for _ in range(20):
                m.step_async(xp, yp)
            torch.cuda.synchronize()
            e0, e1 = _events()
            e0.record()
            for _ in range(steps):
                l = m.step_async(xp, yp)
            e1.record()
            torch.cuda.synchronize()
            nv.check_status()
            rec["b200_graph_step_ms"] = e0.elapsed_time(e1) / steps
            rec["b200_launches_per_step"] = getattr(m.trainer, "launches_per_step", None)
            rec["loss_first"], rec["loss_last"] = first, float(l)
        rows.append(rec)
    print(json.dumps({"config": "ref_mlp", "steps": steps, "rows": rows}), flush=True)


def run_attention(args):
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops import functional as F
    from rust_neural_network_b200.ops import linear_attention as LA
    from rust_neural_network_b200.utils.kernel_bench import time_fn

    dev = torch.device("cuda", 0)
    B, H, S, d = args.batch or 8, 16, args.seq or 4096, args.head_dim
    torch.manual_seed(0)
    q, k, v = (torch.randn(B, S, H, d, device=dev).bfloat16().requires_grad_(True) for _ in range(3))
    w = torch.randn(B, S, H, d, device=dev).bfloat16()
    out = {"config": "attention", "batch": B, "heads": H, "seq": S, "head_dim": d, "dtype": "bf16", "l2_policy": "L2 flushed between iterations"}

    def fb(fn):
        def run():
            for t in (q, k, v):
                t.grad = None
            fn().backward(w)
        return run

    flops_flash = 4.0 * B * H * S * S * d / 2 * 3.5                     # causal: forward 1x, backward 2.5x of 4 S^2 d / 2
    ms = time_fn(fb(lambda: F.flash_attention(q, k, v, causal=True)), args.iters)
    out["flash_causal_fwd_bwd_ms"] = ms
    out["flash_tflops"] = flops_flash / ms / 1e9
    for kind in ("elu", "relu2"):
        ms = time_fn(fb(lambda: LA.linear_attention(q, k, v, kind=kind, causal=True)), args.iters)
        out[f"linear_{kind}_causal_fwd_bwd_ms"] = ms
    nv.check_status()
    print(json.dumps(out), flush=True)


def run_attention_sp(args):
    """Causal linear attention over a sequence sharded across the ranks (launch under torch.distributed.run): every rank
    holds seq / world tokens; only the d x (d + 8) KV states cross NVLink (one fused exchange kernel per direction)."""
    import torch.distributed as dist
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops import linear_attention as LA
    from rust_neural_network_b200.parallel.sp import SPContext

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    B, H, S, d = args.batch or 8, 16, args.seq or 65536, args.head_dim
    s_loc = S // world
    torch.manual_seed(rank)
    q, k, v = (torch.randn(B, s_loc, H, d, device=dev).bfloat16().requires_grad_(True) for _ in range(3))
    w = torch.randn(B, s_loc, H, d, device=dev).bfloat16()
    sp = SPContext(B * H * d * (d + 8), device=dev, backend="fused")
    out = {"config": "attention_sp", "n_gpus": world, "batch": B, "heads": H, "seq": S, "seq_per_gpu": s_loc, "head_dim": d, "dtype": "bf16"}
    for kind in ("elu", "relu2"):
        def step():
            for t in (q, k, v):
                t.grad = None
            LA.linear_attention(q, k, v, kind=kind, causal=True, sp=sp).backward(w)
        for _ in range(3):
            step()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = _events()
        e0.record()
        for _ in range(args.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[f"linear_{kind}_causal_fwd_bwd_ms"] = float(t.item())
    nv.check_status()
    if rank == 0:
        print(json.dumps(out), flush=True)
    sys.stdout.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=["mlp", "ref_mlp", "looped_lm", "moe_lm", "mamba_lm", "attention", "attention_sp"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the preset's layer count (diagnostics)")
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--impl", default="b200", choices=["b200", "torch"], help="torch: the NCCL + cuBLAS library arm (moe_lm, mamba_lm)")
    ap.add_argument("--parallel", default="auto", choices=["auto", "dp", "tp", "ep"], help="layout for N > 1 (auto: the preset's)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"], help="b200 arm: fused peer-memory kernels or NCCL calls")
    ap.add_argument("--recompute-scan", action="store_true", help="mamba_lm: rebuild the scan checkpoints in the backward (less memory, one more forward scan per layer)")
    ap.add_argument("--kernel-table", default="", help="after timing, profile one more step and write device time per kernel name here")
    ap.add_argument("--buckets", action="store_true", help="dp: bucketed gradient reduction overlapped with backward")
    args = ap.parse_args()
    if args.config == "mlp":
        run_mlp(args)
    elif args.config == "ref_mlp":
        run_ref_mlp(args)
    elif args.config == "attention":
        run_attention(args)
    elif args.config == "attention_sp":
        run_attention_sp(args)
    elif args.impl == "torch":
        run_lm_torch(args.config, args)
    else:
        run_lm(args.config, args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
