"""Worker launched by the data-parallel tests (one process per rank, via torch.distributed.run).

Every rank builds the same small LM from the same seed, trains a few steps on ITS slice of a fixed
global batch with `DistributedAdam`, and rank 0 compares the resulting weights against a
single-process run over the whole batch (the oracle: averaging per-rank mean gradients equals the
gradient of the mean over the global batch). `--mode fused` exercises the fused
reduce-scatter + Adam + all-gather kernel over peer memory, `--mode nccl` the all-reduce baseline;
on CPU ranks (gloo) only the baseline path exists.
"""
import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def build(device, dtype):
    from rust_neural_network_b200.models.lm import LoopedTransformerLM
    torch.manual_seed(42)
    m = LoopedTransformerLM(vocab=256, d_model=128, heads=2, ff_dim=256, layers_per_block=1, loops=2, max_seq=128, causal=True)
    return m.to_device(device, dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="fused")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--multimem", type=int, default=0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.device == "cuda":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype = torch.float32
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.parallel.ddp import DistributedAdam

    g = torch.Generator().manual_seed(7)
    gb = 2 * world
    ids = torch.randint(0, 256, (gb, 128), generator=g)
    lab = torch.randint(0, 256, (gb, 128), generator=g)
    per = gb // world

    model = build(dev, dtype)
    opt = DistributedAdam(model.parameters(), lr=1e-3, mode=args.mode, use_multimem=bool(args.multimem))
    losses = []
    for _ in range(args.steps):
        opt.zero_grad()
        l = model.loss(ids[rank * per:(rank + 1) * per].to(dev), lab[rank * per:(rank + 1) * per].to(dev))
        l.backward()
        opt.step()
        losses.append(float(l))
    if dev.type == "cuda":
        torch.cuda.synchronize()
        nv.check_status()
    opt.gather_master()
    result = {"rank": rank, "losses": losses, "mode": opt.mode, "world": world}
    if rank == 0:
        ref = build(dev, dtype)
        ropt = Adam(ref.parameters(), lr=1e-3)
        for _ in range(args.steps):
            ropt.zero_grad()
            ref.loss(ids.to(dev), lab.to(dev)).backward()
            ropt.step()
        num = den = 0.0
        for p, q in zip(model.parameters(), ref.parameters()):
            num += float((p.detach().float() - q.detach().float()).pow(2).sum())
            den += float(q.detach().float().pow(2).sum())
        result["rel_weight_err"] = (num / max(den, 1e-30)) ** 0.5
        upd = 0.0
        fresh = build(dev, dtype)
        for p, q in zip(fresh.parameters(), ref.parameters()):
            upd += float((p.detach().float() - q.detach().float()).pow(2).sum())
        result["rel_update_size"] = (upd / max(den, 1e-30)) ** 0.5
        # shadows on every rank must equal the bf16 cast of the master weights
        if dev.type == "cuda":
            sh = opt.flat.shadow.float(); ma = opt.flat.master
            result["shadow_err"] = float((sh - ma.bfloat16().float()).abs().max())
    # all ranks must hold identical bf16 weights after the step
    if dev.type == "cuda":
        mine = opt.flat.shadow.float().clone()
        other = mine.clone()
        dist.broadcast(other, src=0)
        result["shadow_mismatch_vs_rank0"] = float((mine - other).abs().max())
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        out = {"ranks": gathered}
        print(json.dumps(out), flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
