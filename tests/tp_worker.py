"""Worker launched by the tensor- / expert-parallel tests (one process per GPU, via torch.distributed.run).

Checks, on every rank, the fused all-gather->GEMM and GEMM->reduce-scatter kernels against the
unsharded GEMM, and the expert-parallel MoE layer (dispatch / combine over peer memory) against the
same layer holding all experts locally. Also times the fused kernels against the NCCL + GEMM baseline
with CUDA events (max over ranks). Rank 0 prints one JSON line.
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


def timed(fn, iters, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)       # global rows M
    ap.add_argument("--kdim", type=int, default=512)
    ap.add_argument("--ncols", type=int, default=2048)          # global N of the column-parallel layer
    ap.add_argument("--iters", type=int, default=0)         # > 0: also time fused vs baseline
    ap.add_argument("--moe", type=int, default=1)
    ap.add_argument("--copy-ctas", type=int, default=0)        # 0: the context's own choice
    ap.add_argument("--copy-sweep", default="")             # e.g. "16,32,64,96": time all-gather -> GEMM at each gather-CTA count
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops import gemm as G
    from rust_neural_network_b200.parallel.tp import TPContext
    nv.cuda()

    M, K, N = args.rows, args.kdim, args.ncols
    g = torch.Generator().manual_seed(7)
    X = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)          # identical on every rank
    W1 = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)        # column-parallel: split N
    b1 = torch.randn(N, generator=g).to(dev)
    W2 = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).to(dev)        # row-parallel: split its K (= N)
    b2 = torch.randn(K, generator=g).to(dev)
    R = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    rows_local, n_local = M // world, N // world
    xs = X[rank * rows_local:(rank + 1) * rows_local].contiguous()
    w1s, b1s = W1[rank * n_local:(rank + 1) * n_local].contiguous(), b1[rank * n_local:(rank + 1) * n_local].contiguous()
    w2s = W2[:, rank * n_local:(rank + 1) * n_local].contiguous()

    out = {"rank": rank, "world": world}
    ctx = TPContext(M, max(K, n_local), max(K, n_local), device=dev, backend="fused", copy_ctas=args.copy_ctas)
    base = TPContext(M, K, N, device=dev, backend="nccl")

    # ---- all-gather -> GEMM (+bias, GELU): h[M, n_local]
    want_h = G.gemm(X, w1s, bias=b1s, act="gelu")
    for it in range(3):                                     # repeated calls exercise the epoch / flag reuse
        h = ctx.all_gather_gemm(xs, w1s, bias=b1s, act="gelu")
    torch.cuda.synchronize()
    nv.check_status()
    out["ag_gemm_rel_err"] = rel(h, want_h)
    out["ag_gemm_vs_baseline"] = rel(h, base.all_gather_gemm(xs, w1s, bias=b1s, act="gelu"))

    # ---- GEMM -> reduce-scatter (+bias, +residual): y[rows_local, K]
    full = G.gemm(want_h_full(G, X, W1, b1), W2, bias=b2, out_dtype=torch.float32) + R.float()
    want_y = full[rank * rows_local:(rank + 1) * rows_local]
    res = R[rank * rows_local:(rank + 1) * rows_local].contiguous()
    for it in range(3):
        y = ctx.gemm_reduce_scatter(h, w2s, bias=b2, residual=res)
    torch.cuda.synchronize()
    nv.check_status()
    out["gemm_rs_rel_err"] = rel(y, want_y)
    out["gemm_rs_vs_baseline"] = rel(y, base.gemm_reduce_scatter(h, w2s, bias=b2, residual=res))

    if args.iters > 0:
        mine = ctx.ag_input(rows_local, K)
        mine.copy_(xs)
        out["ms_ag_gemm_fused"] = timed(lambda: ctx.all_gather_gemm(mine, w1s, bias=b1s, act="gelu"), args.iters, dev)
        if args.copy_sweep:
            sweep, keep = {}, ctx.copy_ctas
            for c in (int(v) for v in args.copy_sweep.split(",")):
                ctx.copy_ctas = c
                got = ctx.all_gather_gemm(mine, w1s, bias=b1s, act="gelu")
                sweep[str(c)] = {"ms": timed(lambda: ctx.all_gather_gemm(mine, w1s, bias=b1s, act="gelu"), args.iters, dev), "rel_err": rel(got, want_h)}
            ctx.copy_ctas = keep
            out["ag_gemm_copy_sweep"] = sweep
        out["ms_ag_gemm_nccl"] = timed(lambda: base.all_gather_gemm(xs, w1s, bias=b1s, act="gelu"), args.iters, dev)
        out["ms_gemm_rs_fused"] = timed(lambda: ctx.gemm_reduce_scatter(h, w2s, bias=b2, residual=res), args.iters, dev)
        out["ms_gemm_rs_nccl"] = timed(lambda: base.gemm_reduce_scatter(h, w2s, bias=b2, residual=res), args.iters, dev)
        out["ms_gemm_local_col"] = timed(lambda: G.gemm(X, w1s, bias=b1s, act="gelu"), args.iters, dev)
        out["ms_gemm_local_row"] = timed(lambda: G.gemm(h, w2s), args.iters, dev)
        nv.check_status()

    # ---- differentiable sharded MLP (forward + backward = four fused kernels) against the unsharded layers
    if args.moe:
        from rust_neural_network_b200.parallel.tp import TensorParallelMLP
        Mm, dm, hm = world * 256, 256, 1024
        gm = torch.Generator().manual_seed(21)
        Xm = (torch.randn(Mm, dm, generator=gm) * 0.5).to(torch.bfloat16).to(dev)
        Wa, ba = torch.randn(hm, dm, generator=gm) * 0.05, torch.randn(hm, generator=gm) * 0.1
        Wb, bb = torch.randn(dm, hm, generator=gm) * 0.05, torch.randn(dm, generator=gm) * 0.1
        GYm = torch.randn(Mm, dm, generator=gm).to(torch.bfloat16).to(dev)
        ref_p = [t.to(dev).float().requires_grad_(True) for t in (Wa, ba, Wb, bb)]
        xr = Xm.float().requires_grad_(True)
        yr = xr + torch.nn.functional.gelu(xr @ ref_p[0].t() + ref_p[1], approximate="tanh") @ ref_p[2].t() + ref_p[3]
        yr.backward(GYm.float())
        mctx = TPContext(Mm, hm, hm, device=dev, backend="fused")
        mlp = TensorParallelMLP(dm, hm, mctx, act="gelu", w1=Wa, b1=ba, w2=Wb, b2=bb)
        rl, hl = Mm // world, hm // world
        xs_m = Xm[rank * rl:(rank + 1) * rl].clone().requires_grad_(True)
        for _ in range(2):                                   # twice: staging halves and epochs alternate
            for t in [xs_m] + mlp.parameters():
                t.grad = None
            ym = mlp(xs_m)
            ym.backward(GYm[rank * rl:(rank + 1) * rl])
        torch.cuda.synchronize()
        nv.check_status()
        out["tpmlp_fwd_rel_err"] = rel(ym, yr[rank * rl:(rank + 1) * rl])
        out["tpmlp_dx_rel_err"] = rel(xs_m.grad, xr.grad[rank * rl:(rank + 1) * rl])
        out["tpmlp_dW1_rel_err"] = rel(mlp.up.weight.grad, ref_p[0].grad[rank * hl:(rank + 1) * hl])
        out["tpmlp_db1_rel_err"] = rel(mlp.up.bias.grad, ref_p[1].grad[rank * hl:(rank + 1) * hl])
        out["tpmlp_dW2_rel_err"] = rel(mlp.down.weight.grad, ref_p[2].grad[:, rank * hl:(rank + 1) * hl])
        out["tpmlp_db2_rel_err"] = rel(mlp.down.bias.grad, ref_p[3].grad)

    # ---- expert parallelism: dispatch / combine over peer memory
    if args.moe:
        from rust_neural_network_b200.models.moe import FineGrainedMoE
        E, d, hid, T = 8, 256, 512, 1024
        torch.manual_seed(11)
        full_moe = FineGrainedMoE(d, hid, hid, E, top_k=2, num_shared=1, capacity_factor=8.0, act="silu").to_device(dev, torch.bfloat16)
        torch.manual_seed(11)
        ep_moe = FineGrainedMoE(d, hid, hid, E, top_k=2, num_shared=1, capacity_factor=8.0, act="silu", ep_group=dist.group.WORLD).to_device(dev, torch.bfloat16)
        e_local = E // world
        with torch.no_grad():
            for name in ("W1", "b1", "W2", "b2"):
                getattr(ep_moe, name).data.copy_(getattr(full_moe, name).data[rank * e_local:(rank + 1) * e_local])
            for pa, pb in zip(ep_moe.gate.parameters() + ep_moe.shared[0].parameters(), full_moe.gate.parameters() + full_moe.shared[0].parameters()):
                pa.data.copy_(pb.data)
        gx = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(T, d, generator=gx).to(torch.bfloat16).to(dev).requires_grad_(True)
        x2 = x.detach().clone().requires_grad_(True)
        yo = ep_moe(x)
        yr = full_moe(x2)
        gy = torch.randn(T, d, generator=gx).to(torch.bfloat16).to(dev)
        yo.backward(gy)
        yr.backward(gy)
        torch.cuda.synchronize()
        nv.check_status()
        out["ep_fwd_rel_err"] = rel(yo, yr)
        out["ep_dx_rel_err"] = rel(x.grad, x2.grad)
        # expert weight gradients: the EP rank sees tokens of ALL ranks, the local model only its own -> sum over ranks
        gfull = full_moe.W1.grad.float().clone()
        dist.all_reduce(gfull)
        out["ep_dW1_rel_err"] = rel(ep_moe.W1.grad, gfull[rank * e_local:(rank + 1) * e_local])

    # ---- sequence-parallel linear attention: only the KV states cross ranks
    if args.moe:
        from rust_neural_network_b200.ops.linear_attention import linear_attention
        from rust_neural_network_b200.parallel.sp import SPContext
        B, S_loc, H, d = 2, 512, 4, 64
        gq = torch.Generator().manual_seed(5)
        full = [(torch.randn(B, S_loc * world, H, d, generator=gq) * 0.5).to(torch.bfloat16).to(dev) for _ in range(3)]
        gfull = (torch.randn(B, S_loc * world, H, d, generator=gq)).to(torch.bfloat16).to(dev)
        sp = SPContext(B * H * d * (d + 8), device=dev, backend="fused")
        for causal in (True, False):
            ref_in = [t.clone().requires_grad_(True) for t in full]
            ref = linear_attention(*ref_in, scale=0.125, causal=causal)
            ref.backward(gfull)
            sl = slice(rank * S_loc, (rank + 1) * S_loc)
            loc_in = [t[:, sl].clone().requires_grad_(True) for t in full]
            got = linear_attention(*loc_in, scale=0.125, causal=causal, sp=sp)
            got.backward(gfull[:, sl])
            torch.cuda.synchronize()
            nv.check_status()
            tag = "causal" if causal else "full"
            # fp32 O(S^2) oracle: the sharded run must be as close to it as the unsharded bf16 run is
            from rust_neural_network_b200.ops.linear_attention import linear_attention_ref
            orc_in = [t.float().clone().requires_grad_(True) for t in full]
            orc = linear_attention_ref(*orc_in, scale=0.125, causal=causal)
            orc.backward(gfull.float())
            out[f"sp_{tag}_fwd_rel_err"] = rel(got, orc[:, sl])
            out[f"ref_{tag}_fwd_rel_err"] = rel(ref[:, sl], orc[:, sl])
            for i, nm in enumerate(("dq", "dk", "dv")):
                out[f"sp_{tag}_{nm}_rel_err"] = rel(loc_in[i].grad, orc_in[i].grad[:, sl])
                out[f"ref_{tag}_{nm}_rel_err"] = rel(ref_in[i].grad[:, sl], orc_in[i].grad[:, sl])

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
    torch.cuda.synchronize()
    dist.destroy_process_group()


def want_h_full(G, X, W1, b1):
    return G.gemm(X, W1, bias=b1, act="gelu")


if __name__ == "__main__":
    main()
