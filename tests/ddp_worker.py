"""Worker launched by the data-parallel tests (one process per rank, via torch.distributed.run).

Every rank builds the same small LM from the same seed, trains a few steps on ITS slice of a fixed
global batch with `DistributedAdam` / `DistributedMuon`, and rank 0 compares the resulting weights against a
single-process run over the whole batch (the oracle: averaging per-rank mean gradients equals the
gradient of the mean over the global batch). `--mode fused` exercises the fused reduce-scatter +
optimizer + all-gather kernels over peer memory, `--mode nccl` the all-reduce baseline; on CPU ranks
(gloo) only the baseline path exists.

Options: `--opt muon` (per-tensor RMS rule), `--clip X` (global-norm clipping of the averaged gradient),
`--groups 1` (bucketed launches from the model's marks, overlapping backward), `--graph 1` (the whole step
replayed as a CUDA graph through `Trainer`, with rank 1 delayed before every replay, compared against the
eager distributed run), `--ckpt DIR` (collective checkpoint save; the test reloads it under another world size).
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
    m = LoopedTransformerLM(vocab=512, d_model=128, heads=2, ff_dim=256, layers_per_block=1, loops=2, max_seq=128, causal=True)
    return m.to_device(device, dtype)


def make_opt(model, args, world_kind):
    from rust_neural_network_b200.optim import Adam, Muon
    from rust_neural_network_b200.parallel.ddp import DistributedAdam, DistributedMuon
    clip = args.clip if args.clip > 0 else None
    if world_kind == "single":
        return Adam(model.parameters(), lr=1e-3) if args.opt == "adam" else Muon(model.parameters(), lr=1e-3, momentum=0.9)
    kw = dict(mode=args.mode, use_multimem=bool(args.multimem), groups=model.dp_groups() if args.groups else None, bucket_mb=0.05,
              replicate_max_numel=1024)        # at this size only biases / norm gains stay replicated: the matrices are sharded
    if args.opt == "adam":
        return DistributedAdam(model.parameters(), lr=1e-3, max_grad_norm=clip, **kw)
    return DistributedMuon(model.parameters(), lr=1e-3, momentum=0.9, **kw)


def sq(t):
    return float(t.detach().float().pow(2).sum())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="fused")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--multimem", type=int, default=0)
    ap.add_argument("--opt", default="adam")
    ap.add_argument("--clip", type=float, default=0.0)
    ap.add_argument("--groups", type=int, default=0)
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--ckpt", default="")
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
    from rust_neural_network_b200.parallel.ddp import is_replicated
    from rust_neural_network_b200.train import Trainer

    g = torch.Generator().manual_seed(7)
    gb = 2 * world
    ids = torch.randint(0, 512, (gb, 128), generator=g)
    lab = torch.randint(0, 512, (gb, 128), generator=g)
    per = gb // world
    my_ids, my_lab = ids[rank * per:(rank + 1) * per], lab[rank * per:(rank + 1) * per]
    clip = args.clip if args.clip > 0 else None

    def run_eager(model, opt, x, y, steps):
        losses = []
        for _ in range(steps):
            opt.zero_grad()
            l = model.loss(x.to(dev), y.to(dev))
            l.backward()
            if clip is not None:
                opt.clip_grad_norm(clip)
            opt.step()
            losses.append(float(l))
        return losses

    model = build(dev, dtype)
    opt = make_opt(model, args, "dist")
    losses = run_eager(model, opt, my_ids, my_lab, args.steps)
    if dev.type == "cuda":
        torch.cuda.synchronize()
        nv.check_status()
    result = {"rank": rank, "losses": losses, "mode": opt.mode, "world": world, "buckets": len(opt.buckets),
              "norm": float(opt._scalars[2]) if clip is not None else None}

    # ---- values the forward consumes must be bit-identical on all ranks BEFORE any gather: the bf16 shadow
    # everywhere and the fp32 master of every replicated parameter
    if dev.type == "cuda" and opt.mode == "fused":
        mine = opt.flat.shadow.float().clone(); other = mine.clone()
        dist.broadcast(other, src=0)
        result["shadow_mismatch_vs_rank0"] = float((mine - other).abs().max())
        rep = opt.flat.master[opt.n_shard:].clone(); other = rep.clone()
        dist.broadcast(other, src=0)
        result["replicated_master_mismatch_vs_rank0"] = float((rep - other).abs().max()) if rep.numel() else 0.0
        result["n_replicated"] = int(rep.numel())

    if args.ckpt:
        from rust_neural_network_b200.serialize import save_checkpoint
        save_checkpoint(os.path.join(args.ckpt, "dp.rnnb"), model, opt)
    opt.gather_master()

    # ---- graph replay with a delayed rank against the eager distributed run
    if args.graph and dev.type == "cuda":
        from rust_neural_network_b200.parallel import ddp as _ddp
        model_g = build(dev, dtype)
        opt_g = make_opt(model_g, args, "dist")
        tr = Trainer(model_g, opt_g, loss_fn=None, use_cuda_graph=True, grad_clip=clip)
        for _ in range(args.steps):
            if rank == 1:
                torch.cuda._sleep(int(40e6))             # tens of ms: peers must really wait for this rank's gradients
            tr.train_step(my_ids, my_lab)
        torch.cuda.synchronize()
        nv.check_status()
        opt_g.gather_master()
        num = sum(sq(p - q) for p, q in zip(model_g.parameters(), model.parameters()))
        result["graph_vs_eager_sq"] = num
        _ddp._ACTIVE = opt

    if rank == 0:
        ref = build(dev, dtype)
        ropt = make_opt(ref, args, "single")
        run_eager(ref, ropt, ids, lab, args.steps)
        # a parameter whose gradient is rounding noise (the key bias: softmax ignores a shift along the keys) gets an
        # Adam update of full size in a random direction; it cannot be compared parameter by parameter
        # (judged on an fp32 CPU copy of the model, where that noise is ~1e-11 instead of bf16's ~1e-6)
        cref = build(torch.device("cpu"), torch.float32)
        cref.loss(ids, lab).backward()
        noise = [q.grad is None or float(q.grad.abs().max()) < 1e-7 for q in cref.parameters()]
        fresh = build(dev, dtype)
        num = den = upd = 0.0
        rep_num = rep_upd = 0.0
        worst_rep = 0.0
        for p, q, f, nz in zip(model.parameters(), ref.parameters(), fresh.parameters(), noise):
            if nz:
                continue
            e, u = sq(p - q), sq(f - q)
            num += e; den += sq(q); upd += u
            if opt.is_rep(p):
                rep_num += e; rep_upd += u
                if u > 0:
                    worst_rep = max(worst_rep, (e / u) ** 0.5)
        result["rel_weight_err"] = (num / max(den, 1e-30)) ** 0.5
        result["rel_update_size"] = (upd / max(den, 1e-30)) ** 0.5
        result["err_over_update"] = (num / max(upd, 1e-30)) ** 0.5
        result["replicated_err_over_update"] = (rep_num / max(rep_upd, 1e-30)) ** 0.5
        result["worst_replicated_param_err_over_update"] = worst_rep
        if "graph_vs_eager_sq" in result:
            result["graph_vs_eager_over_update"] = (result["graph_vs_eager_sq"] / max(upd, 1e-30)) ** 0.5
        if dev.type == "cuda":
            sh = opt.flat.shadow.float(); ma = opt.flat.master
            result["shadow_err"] = float((sh - ma.bfloat16().float()).abs().max())
        if args.ckpt:
            from rust_neural_network_b200.serialize import save_checkpoint
            save_checkpoint(os.path.join(args.ckpt, "single.rnnb"), ref, ropt)
    if dev.type == "cuda":
        from rust_neural_network_b200.parallel import ddp as D
        torch.cuda.synchronize()
        dist.barrier()                                            # every peer has finished writing into this rank's buffers
        result["canaries_checked"] = D.check_canaries()
        bufs = list(D._LIVE_BUFFERS or ())
        if bufs:                                                  # the detector itself: a byte of a guard band changed on the host side
            raw = bufs[0]._raw.view(torch.uint8)
            keep = int(raw[3])
            raw[3] = 0
            try:
                D.check_canaries()
                result["canary_detects"] = False
            except RuntimeError:
                result["canary_detects"] = True
            raw[3] = keep
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
