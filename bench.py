#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the looped-transformer LM configuration.

Config (fixed): d_model 512, 8 heads x head_dim 64, shared block of 4 pre-norm layers looped 6 times,
GELU FFN 2048, causal FlashAttention, vocab 32000, seq 1024, GLOBAL batch 64 (strong scaling: the
per-GPU batch is 64/N), bf16 compute with fp32 master weights, Adam, N(0, 0.02) init, synthetic
uniform token ids. Every timed step is a full forward + backward + optimizer step; with N > 1 the
gradients are reduced and the update applied by the fused data-parallel kernel path.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events around the K steps, max over
ranks); `e2e.value` is the same metric through `Trainer.train_step` including, every step, the
host->device copy of that step's token ids / labels from pinned memory and a device->host read of
the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

CONFIG = dict(vocab=32000, d_model=512, heads=8, ff_dim=2048, layers_per_block=4, loops=6, seq_len=1024, global_batch=64)
METRIC = "train tokens/s (looped-transformer LM, device-timed, max over ranks)"


def model_flops_per_token(cfg) -> float:
    """Forward + backward FLOPs per token: 6 x the matmul parameters a token passes through (every application of the
    shared block counts) plus causal attention (QK^T and PV, half the square, backward = 2 x forward)."""
    d, ff, S = cfg["d_model"], cfg["ff_dim"], cfg["seq_len"]
    apps = cfg["layers_per_block"] * cfg["loops"]
    matmul_params = apps * (4 * d * d + 2 * d * ff) + d * cfg["vocab"]
    attn_fwd = apps * 2 * S * d                       # 2 products x 2 FLOP x S x d / 2 (causal)
    return 6.0 * matmul_params + 3.0 * attn_fwd


def sustained_peak_tflops():
    """(peak, source): the sustained bf16 GEMM throughput measured on this pool (MEASURED_PEAKS.json next to this file)
    or, when that file is absent, 1400 TFLOP/s from an earlier measurement."""
    f = Path(__file__).resolve().parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(f.read_text())["bf16_tflops_sustained"]), "of measured"
    except Exception:
        return 1400.0, "of fallback"


def reference_arm(args):
    # The reference is a Rust crate (Cargo.toml, no setup.py / pyproject.toml): pip cannot install it and
    # there is no cargo / rustc in this image, so it cannot be built or run here.
    if int(os.environ.get("RANK", "0")) != 0:          # under torch.distributed.run only rank 0 reports
        return 0
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a Rust crate: pip install fails (no setup.py/pyproject.toml) and no cargo/rustc toolchain is available offline",
                      "metric": METRIC, "n_gpus": args.gpus}))
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self._stop_evt, self.proc = index, [], threading.Event(), None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            for line in self.proc.stdout:
                if self._stop_evt.is_set():
                    break
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
        except Exception:
            pass

    def stop(self):
        self._stop_evt.set()
        if self.proc is not None:
            try:
                self.proc.terminate()
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        for p in self.samples:
            try:
                sm.append(float(p[0])); mx = max(mx, float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def torch_arm(args, in_process: bool = False):
    """The library baseline: same model, shapes, precision policy and timing rules, stock PyTorch kernels only.
    `in_process`: called from the b200 arm after its own measurement (the process group exists already); returns the
    record instead of printing it."""
    import torch
    import torch.distributed as dist
    from baseline.torch_lm import TorchLoopedLM, TorchStep

    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0")); local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(CONFIG)
    if args.small:
        cfg.update(vocab=2048, d_model=128, heads=2, ff_dim=256, layers_per_block=2, loops=2, seq_len=256, global_batch=8)
    if args.global_batch > 0:
        cfg["global_batch"] = args.global_batch
    local_batch, S = cfg["global_batch"] // world, cfg["seq_len"]
    torch.manual_seed(1234)
    model = TorchLoopedLM(cfg["vocab"], cfg["d_model"], cfg["heads"], cfg["ff_dim"], cfg["layers_per_block"], cfg["loops"], S).to(dev)
    step = TorchStep(model, local_batch, S, dev, world, graph=not args.no_graph)
    g = torch.Generator().manual_seed(1000 + rank)
    pool = 4
    host_ids = [torch.randint(0, cfg["vocab"], (local_batch, S), generator=g).pin_memory() for _ in range(pool)]
    host_lab = [torch.randint(0, cfg["vocab"], (local_batch, S), generator=g).pin_memory() for _ in range(pool)]
    dev_ids, dev_lab = [t.to(dev) for t in host_ids], [t.to(dev) for t in host_lab]
    step.ids.copy_(dev_ids[0]); step.labels.copy_(dev_lab[0])
    step.warmup(args.warmup)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start(); time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step.step_device(dev_ids[i % pool], dev_lab[i % pool])
    e1.record()
    barrier()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    last = 0.0
    for i in range(args.steps):
        last = float(step.step_device(host_ids[i % pool], host_lab[i % pool]).item())
    t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1))
    if in_process:
        if rank == 0:
            sampler.stop()
        tokens = cfg["global_batch"] * S * args.steps
        del step, model
        torch.cuda.empty_cache()
        return {"value": tokens / (dev_ms / 1e3), "ms_per_step": dev_ms / args.steps, "e2e_value": tokens / (e2e_ms / 1e3),
                "e2e_ms_per_step": e2e_ms / args.steps, "loss_last": last}
    if rank == 0:
        sampler.stop()
        tokens = cfg["global_batch"] * S * args.steps
        print(json.dumps({
            "metric": METRIC, "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init N(0,0.02) weights", "impl": "torch",
            "config": {"model": "looped-transformer LM d512 h8 hd64, 4 layers x 6 loops, ff2048, vocab32000 (stock PyTorch: cuBLAS, SDPA, fused Adam, DDP)",
                       "global_batch": cfg["global_batch"], "seq_len": S, "parallelism": f"dp{world}" + ("-ddp-nccl" if world > 1 else ""),
                       "l2_policy": "inputs larger than L2 (multi-GB activation working set per step)", "cuda_graph": step.graph is not None,
                       "small": bool(args.small)},
            "clocks": sampler.summary(),
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": host_ids[0].numel() * 8 * 2, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "loss_last": last}), flush=True)
    if world > 1:
        barrier()
        sys.stdout.flush()
        os._exit(0)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "torch"],
                    help="b200: this package; reference: the unmodified upstream; torch: stock PyTorch (cuBLAS, SDPA, fused Adam, DDP) on the same model")
    ap.add_argument("--no-graph", action="store_true", help="run eagerly instead of replaying a captured CUDA graph")
    ap.add_argument("--dp", default="fused", choices=["fused", "nccl"], help="data-parallel gradient path for N > 1")
    ap.add_argument("--global-batch", type=int, default=0, help="override the global batch (diagnostics; the headline configuration is 64)")
    ap.add_argument("--small", action="store_true", help="tiny configuration for smoke tests (NOT a valid bench number)")
    ap.add_argument("--no-pair", action="store_true", help="bf16 GEMMs on single-CTA tiles only, no CTA pairs (diagnostics)")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (diagnostics)")
    ap.add_argument("--no-torch-arm", action="store_true", help="skip the stock-PyTorch run that follows the measurement (the `torch_arm` / `vs_torch` keys)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "torch":
        return torch_arm(args)

    import torch
    import torch.distributed as dist
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.models.lm import LoopedTransformerLM
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.train import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    nv.cuda()
    if args.no_pdl:
        nv.set_pdl(False)
    if args.no_pair:
        nv.set_gemm_pair(False)

    cfg = dict(CONFIG)
    if args.small:
        cfg.update(vocab=2048, d_model=128, heads=2, ff_dim=256, layers_per_block=2, loops=2, seq_len=256, global_batch=8)
    if args.global_batch > 0:
        cfg["global_batch"] = args.global_batch
    assert cfg["global_batch"] % world == 0
    local_batch = cfg["global_batch"] // world
    S = cfg["seq_len"]

    torch.manual_seed(1234)          # identical initial weights on every rank
    model = LoopedTransformerLM(cfg["vocab"], cfg["d_model"], cfg["heads"], cfg["ff_dim"], cfg["layers_per_block"],
                                cfg["loops"], S, causal=True).to_device(dev, dtype=torch.bfloat16)
    if world > 1:
        from rust_neural_network_b200.parallel.ddp import DistributedAdam
        opt = DistributedAdam(model.parameters(), lr=1e-3, mode=args.dp)
    else:
        opt = Adam(model.parameters(), lr=1e-3)
    trainer = Trainer(model, opt, loss_fn=None, use_cuda_graph=not args.no_graph)

    # synthetic data: a pool of pinned host batches (uniform token ids), different on every rank
    g = torch.Generator().manual_seed(1000 + rank)
    pool = 4
    host_ids = [torch.randint(0, cfg["vocab"], (local_batch, S), generator=g).pin_memory() for _ in range(pool)]
    host_lab = [torch.randint(0, cfg["vocab"], (local_batch, S), generator=g).pin_memory() for _ in range(pool)]
    h2d_bytes = host_ids[0].numel() * host_ids[0].element_size() * 2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up (also captures the CUDA graph)
    loss0 = None
    for i in range(args.warmup):
        l = trainer.train_step(host_ids[i % pool], host_lab[i % pool])
        if loss0 is None:
            loss0 = float(l)
    torch.cuda.synchronize()
    nv.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    # ---- device-timed region: K steps on device-resident inputs (kernel time only)
    dev_ids = [t.to(dev) for t in host_ids]
    dev_lab = [t.to(dev) for t in host_lab]
    barrier()
    nv.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        if trainer._graph is not None:
            trainer._static[0].copy_(dev_ids[i % pool]); trainer._static[1].copy_(dev_lab[i % pool])
            trainer._graph.replay()
        else:
            trainer._step_device(dev_ids[i % pool], dev_lab[i % pool])
    e1.record()
    barrier()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = (trainer.launches_per_step * args.steps) if trainer._graph is not None else nv.launch_count()

    # ---- end-to-end region: public API, pinned-host inputs copied every step, loss read back every step
    barrier()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    last = 0.0
    for i in range(args.steps):
        loss = trainer.train_step(host_ids[i % pool], host_lab[i % pool])
        last = float(loss.item())          # device -> host read of the step's result
    t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1))
    if rank == 0:
        sampler.stop()
    nv.check_status()

    tokens_per_step = cfg["global_batch"] * S
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    peak, peak_src = sustained_peak_tflops()
    tflops_per_gpu = model_flops_per_token(cfg) * value / world / 1e12
    # the same model on stock PyTorch (cuBLAS, SDPA, fused Adam, DDP), measured in this process right after, same rules
    torch_rec = None
    if not args.no_torch_arm:
        try:
            torch_rec = torch_arm(args, in_process=True)
        except Exception as e:                                   # the headline number does not depend on this arm
            torch_rec = {"error": repr(e)[:200]}
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "impl": "b200",
            "config": {"model": "looped-transformer LM d512 h8 hd64, 4 layers x 6 loops, ff2048, vocab32000",
                       "global_batch": cfg["global_batch"], "seq_len": S,
                       "parallelism": f"dp{world}" + (f"-{args.dp}" if world > 1 else ""),
                       "l2_policy": "inputs larger than L2 (multi-GB activation working set per step)",
                       "cuda_graph": trainer._graph is not None, "pdl": not args.no_pdl, "gemm_cta_pairs": not args.no_pair, "small": bool(args.small)},
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline_pct": 100.0 * tflops_per_gpu / peak,
            "roofline": {"model_gflop_per_token": model_flops_per_token(cfg) / 1e9, "tflops_per_gpu": tflops_per_gpu,
                         "peak_tflops_bf16_sustained": peak, "peak_source": peak_src},
            "torch_arm": torch_rec,
            "vs_torch": (value / torch_rec["value"]) if torch_rec and "value" in torch_rec else None,
            "vs_torch_e2e": (e2e_value / torch_rec["e2e_value"]) if torch_rec and "e2e_value" in torch_rec else None,
            "loss_first": loss0, "loss_last": last,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        # a CUDA graph that captured collective kernels has to be released before its communicator
        barrier()
        trainer._graph = None
        del trainer, opt
        import gc
        gc.collect()
        torch.cuda.synchronize()
        if args.dp == "nccl":
            sys.stdout.flush()
            os._exit(0)          # the communicator's teardown after graph-captured collectives does not return
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
