"""Worker of the model-level parallelism tests (one process per rank, via torch.distributed.run).

`--model mamba_tp`: a tensor-parallel Mamba LM (channel-sharded blocks on row-sharded activations) against the same
model held whole by one process: loss, gradients of sharded and replicated parameters, and a few optimizer steps.
`--model moe_ep`: an expert-parallel MoE transformer LM against the same model with all experts local.
Runs on CPU ranks (gloo; the collectives take their baseline path) and on GPUs (the fused kernels).
"""
import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def gather_cat(t, dim, world):
    parts = [None] * world
    dist.all_gather_object(parts, t.detach().float().cpu())
    return torch.cat(parts, dim)


def mamba_tp(args, rank, world, dev, dtype):
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.models.mamba import MambaLM
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.parallel.tp import TPContext
    V, d, L, N, R, S, Bl = 256, (64 if world <= 4 else 128), 2, 16, 8, 128, 2      # 32 inner channels per rank at least
    di = 2 * d
    M = world * Bl * S
    tp = TPContext(M, d, d, device=dev, backend=args.backend, max_allreduce_numel=M * (R + 2 * N))
    torch.manual_seed(3)                                    # embedding / norms / head: same draw on every rank
    model = MambaLM(V, d, L, d_state=N, dt_rank=R, tp=tp, seed=77).to_device(dev, dtype)
    opt = model.make_optimizer(lr=1e-3)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, V, (world * Bl, S), generator=g)
    lab = torch.randint(0, V, (world * Bl, S), generator=g)
    my = slice(rank * Bl, (rank + 1) * Bl)

    # ---- the same model, whole, on rank 0 (weights gathered from the shards)
    full = {}
    dl = di // world
    for li, b in enumerate(model.blocks):
        inp = b.in_proj.detach().float().cpu()
        full[f"{li}.in_x"] = gather_cat(inp[:dl], 0, world); full[f"{li}.in_z"] = gather_cat(inp[dl:], 0, world)
        full[f"{li}.conv_w"] = gather_cat(b.conv_weight, 0, world); full[f"{li}.conv_b"] = gather_cat(b.conv_bias, 0, world)
        full[f"{li}.a"] = gather_cat(b.a, 0, world); full[f"{li}.xp"] = gather_cat(b.x_proj, 1, world)
        full[f"{li}.dt_up"] = gather_cat(b.dt_up, 0, world); full[f"{li}.dt_bias"] = gather_cat(b.dt_bias, 0, world)
        full[f"{li}.d_skip"] = gather_cat(b.d_skip, 0, world); full[f"{li}.out"] = gather_cat(b.out_proj, 1, world)
    shared0 = [p.detach().clone() for p in model.tok.parameters() + model.ln_final.parameters() + model.lm_head.parameters()]
    out = {"rank": rank, "world": world}

    def tp_step(train):
        opt.zero_grad()
        l = model.loss(ids[my].to(dev), lab[my].to(dev))
        l.backward()
        if train:
            opt.step()
        t = l.detach().float().reshape(1).clone()
        dist.all_reduce(t)
        return float(t) / world

    loss0 = tp_step(False)
    if dev.type == "cuda":
        torch.cuda.synchronize(); nv.check_status()
    grads = {}
    b0 = model.blocks[0]
    inp_g = b0.in_proj.grad.detach().float().cpu()
    grads["in_x"] = gather_cat(inp_g[:dl], 0, world); grads["xp"] = gather_cat(b0.x_proj.grad, 1, world)
    grads["out"] = gather_cat(b0.out_proj.grad, 1, world); grads["a"] = gather_cat(b0.a.grad, 0, world)
    grads["dt_bias"] = gather_cat(b0.dt_bias.grad, 0, world)
    for name, p in (("tok", model.tok.weight), ("ln0_gamma", model.norms[0].gamma), ("head", model.lm_head.weight)):
        t = p.grad.detach().float().clone()
        dist.all_reduce(t)                                   # replicated parameters: the ranks hold partial sums
        grads[name] = t.cpu()
    losses = [tp_step(True) for _ in range(args.steps)]
    if dev.type == "cuda":
        torch.cuda.synchronize(); nv.check_status()
    out["tp_losses"] = [loss0] + losses

    if rank == 0:
        torch.manual_seed(3)
        ref = MambaLM(V, d, L, d_state=N, dt_rank=R).to_device(dev, dtype)
        with torch.no_grad():
            for li, b in enumerate(ref.blocks):
                f = lambda k: full[f"{li}.{k}"].to(dev)
                b.in_proj_x.weight.copy_(f("in_x")); b.in_proj_z.weight.copy_(f("in_z"))
                b.conv_weight.copy_(f("conv_w")); b.conv_bias.copy_(f("conv_b")); b.a.copy_(f("a"))
                xp = f("xp")
                b.proj_delta.weight.copy_(xp[:R]); b.proj_b.weight.copy_(xp[R:R + N]); b.proj_c.weight.copy_(xp[R + N:])
                b.dt_up.weight.copy_(f("dt_up")); b.dt_bias.copy_(f("dt_bias")); b.d_skip.copy_(f("d_skip"))
                b.out_proj.weight.copy_(f("out"))
            for p, q in zip(ref.tok.parameters() + ref.ln_final.parameters() + ref.lm_head.parameters(), shared0):
                p.copy_(q)
        ropt = Adam(ref.parameters(), lr=1e-3)

        def ref_step(train):
            ropt.zero_grad()
            l = ref.loss(ids.to(dev), lab.to(dev))
            l.backward()
            if train:
                ropt.step()
            return float(l)

        r0 = ref_step(False)
        rb = ref.blocks[0]
        want = {"in_x": rb.in_proj_x.weight.grad, "out": rb.out_proj.weight.grad, "a": rb.a.grad, "dt_bias": rb.dt_bias.grad,
                "xp": torch.cat([rb.proj_delta.weight.grad, rb.proj_b.weight.grad, rb.proj_c.weight.grad], 0),
                "tok": ref.tok.weight.grad, "ln0_gamma": ref.norms[0].gamma.grad, "head": ref.lm_head.weight.grad}
        out["grad_rel_err"] = {k: rel(grads[k].to(dev), want[k]) for k in want}
        out["ref_losses"] = [r0] + [ref_step(True) for _ in range(args.steps)]
    return out


def moe_ep(args, rank, world, dev, dtype):
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.models.moe import MoETransformerLM
    from rust_neural_network_b200.optim import Adam
    V, d, L, H, E, k, hid, S, Bl = 256, 128, 2, 2, 8, 2, 128, 128, 2
    torch.manual_seed(3)
    model = MoETransformerLM(V, d, L, H, E, k, 1, hid, S, ep_group=dist.group.WORLD, capacity_factor=float(E),
                             ep_backend=args.backend).to_device(dev, dtype)
    opt = model.make_optimizer(lr=1e-3, mode=args.backend if dev.type == "cuda" else "nccl")
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, V, (world * Bl, S), generator=g)
    lab = torch.randint(0, V, (world * Bl, S), generator=g)
    my = slice(rank * Bl, (rank + 1) * Bl)
    out = {"rank": rank, "world": world}
    experts = {}
    ex_ids = {id(p) for m in model.moe for p in (m.W1, m.b1, m.W2, m.b2)}
    shared0 = [p.detach().clone() for p in model.parameters() if id(p) not in ex_ids]
    for li, m in enumerate(model.moe):
        for nm in ("W1", "b1", "W2", "b2"):
            experts[f"{li}.{nm}"] = gather_cat(getattr(m, nm), 0, world)

    def ep_step(train):
        opt.zero_grad()
        l = model.loss(ids[my].to(dev), lab[my].to(dev))
        l.backward()
        if train:
            opt.step()
        t = l.detach().float().reshape(1).clone()
        dist.all_reduce(t)
        return float(t) / world

    loss0 = ep_step(False)
    if dev.type == "cuda":
        torch.cuda.synchronize(); nv.check_status()
    gW1 = gather_cat(model.moe[0].W1.grad, 0, world) / world     # an expert sums the contributions of every rank's loss
    gate = model.moe[0].gate.weight.grad.detach().float().clone()
    dist.all_reduce(gate)
    gate /= world
    losses = [ep_step(True) for _ in range(args.steps)]
    if dev.type == "cuda":
        torch.cuda.synchronize(); nv.check_status()
    out["ep_losses"] = [loss0] + losses
    if rank == 0:
        torch.manual_seed(3)
        ref = MoETransformerLM(V, d, L, H, E, k, 1, hid, S, capacity_factor=float(E)).to_device(dev, dtype)
        with torch.no_grad():
            for li, m in enumerate(ref.moe):
                for nm in ("W1", "b1", "W2", "b2"):
                    getattr(m, nm).copy_(experts[f"{li}.{nm}"].to(dev))
            def shared(mod):
                ex = {id(p) for m in mod.moe for p in (m.W1, m.b1, m.W2, m.b2)}
                return [p for p in mod.parameters() if id(p) not in ex]
            for p, q in zip(shared(ref), shared0):
                p.copy_(q)
        ropt = Adam(ref.parameters(), lr=1e-3)

        def ref_step(train):
            ropt.zero_grad()
            l = ref.loss(ids.to(dev), lab.to(dev))
            l.backward()
            if train:
                ropt.step()
            return float(l)

        r0 = ref_step(False)
        out["grad_rel_err"] = {"W1": rel(gW1.to(dev), ref.moe[0].W1.grad), "gate": rel(gate.cpu(), ref.moe[0].gate.weight.grad.cpu())}
        out["ref_losses"] = [r0] + [ref_step(True) for _ in range(args.steps)]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mamba_tp")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--backend", default="fused")
    ap.add_argument("--steps", type=int, default=3)
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
    out = {"mamba_tp": mamba_tp, "moe_ep": moe_ep}[args.model](args, rank, world, dev, dtype)
    if torch.cuda.is_available() and dist.get_backend() == "nccl":
        from rust_neural_network_b200.parallel.ddp import check_canaries
        torch.cuda.synchronize()
        dist.barrier()
        out["canaries_checked"] = check_canaries()               # raises if any peer wrote outside a symmetric buffer's payload
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print(json.dumps({"ranks": gathered}), flush=True)
    dist.barrier()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
