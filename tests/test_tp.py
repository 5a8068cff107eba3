"""Tensor- and expert-parallel kernels over NVLink peer memory (2+ GPUs), plus the CPU (gloo) baseline path."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

WORKER = str(Path(__file__).resolve().parent / "tp_worker.py")


def _run(nproc, extra, port, timeout=600):
    env = dict(os.environ)
    env.update({"MASTER_ADDR": "127.0.0.1", "OMP_NUM_THREADS": "2", "NCCL_NVLS_ENABLE": "0"})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('{"ranks"')][-1]
    return json.loads(line)["ranks"]


@pytest.mark.gpu
def test_fused_tp_and_ep_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ranks = _run(2, ["--rows", "4096", "--kdim", "512", "--ncols", "2048"], 29631)
    for r in ranks:
        assert r["ag_gemm_rel_err"] < 1e-2 and r["ag_gemm_vs_baseline"] < 1e-2
        assert r["gemm_rs_rel_err"] < 2e-2 and r["gemm_rs_vs_baseline"] < 2e-2
        assert r["ep_fwd_rel_err"] < 2e-2 and r["ep_dx_rel_err"] < 3e-2 and r["ep_dW1_rel_err"] < 3e-2
        for nm in ("fwd", "dx", "dW1", "db1", "dW2", "db2"):                      # sharded MLP with autograd vs fp32 unsharded
            assert r[f"tpmlp_{nm}_rel_err"] < 3e-2, (nm, r[f"tpmlp_{nm}_rel_err"])
        for tag in ("causal", "full"):
            # against the fp32 oracle: absolute bounds (the causal form runs on the fused kernels with the exchange inside
            # them), and the sequence-sharded run is as accurate as the unsharded bf16 run
            for nm in ("fwd", "dq", "dk", "dv"):
                # dq of the non-causal form: composed bf16 GEMMs with a bf16 global state, 7 % at these sizes
                bound = 1e-2 if nm == "fwd" else ((5e-2 if tag == "causal" else 1e-1) if nm == "dq" else 1.5e-2)
                assert r[f"sp_{tag}_{nm}_rel_err"] < bound, (tag, nm, r[f"sp_{tag}_{nm}_rel_err"])
                assert r[f"sp_{tag}_{nm}_rel_err"] < 1.5 * r[f"ref_{tag}_{nm}_rel_err"] + 5e-3, (tag, nm, r)


def _cpu_tp_rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rust_neural_network_b200.parallel.tp import TPContext
    g = torch.Generator().manual_seed(3)
    X, W1, W2 = torch.randn(8, 6, generator=g), torch.randn(10, 6, generator=g), torch.randn(6, 10, generator=g)
    ctx = TPContext(8, 10, 10, device="cpu", backend="fused")            # CPU ranks always take the baseline path
    h = ctx.all_gather_gemm(X[rank * 4:(rank + 1) * 4], W1[rank * 5:(rank + 1) * 5], act="relu")
    y = ctx.gemm_reduce_scatter(h, W2[:, rank * 5:(rank + 1) * 5].contiguous())
    want = (torch.relu(X @ W1.t()) @ W2.t())[rank * 4:(rank + 1) * 4]
    q.put((rank, float((y.float() - want).abs().max()), float(want.abs().max())))
    dist.destroy_process_group()


def _cpu_tp_mlp_rank(rank, world, port, q):
    """Sharded MLP with autograd against the unsharded computation (forward, input and parameter gradients)."""
    import torch.distributed as dist
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rust_neural_network_b200.parallel.tp import TPContext, TensorParallelMLP
    g = torch.Generator().manual_seed(5)
    M, d, hid = 8, 6, 10
    X, W1, b1 = torch.randn(M, d, generator=g), torch.randn(hid, d, generator=g) * 0.5, torch.randn(hid, generator=g)
    W2, b2, GY = torch.randn(d, hid, generator=g) * 0.5, torch.randn(d, generator=g), torch.randn(M, d, generator=g)
    ref_in = [t.clone().requires_grad_(True) for t in (X, W1, b1, W2, b2)]
    xr, w1r, b1r, w2r, b2r = ref_in
    ref = xr + torch.nn.functional.gelu(xr @ w1r.t() + b1r, approximate="tanh") @ w2r.t() + b2r
    ref.backward(GY)
    ctx = TPContext(M, max(d, hid), max(d, hid), device="cpu")
    mlp = TensorParallelMLP(d, hid, ctx, act="gelu", w1=W1, b1=b1, w2=W2, b2=b2)
    rl, hl = M // world, hid // world
    xs = X[rank * rl:(rank + 1) * rl].clone().requires_grad_(True)
    y = mlp(xs)
    y.backward(GY[rank * rl:(rank + 1) * rl])
    errs = [float((y - ref[rank * rl:(rank + 1) * rl]).abs().max()),
            float((xs.grad - xr.grad[rank * rl:(rank + 1) * rl]).abs().max()),
            float((mlp.up.weight.grad - w1r.grad[rank * hl:(rank + 1) * hl]).abs().max()),
            float((mlp.up.bias.grad - b1r.grad[rank * hl:(rank + 1) * hl]).abs().max()),
            float((mlp.down.weight.grad - w2r.grad[:, rank * hl:(rank + 1) * hl]).abs().max()),
            float((mlp.down.bias.grad - b2r.grad).abs().max())]
    q.put((rank, errs))
    dist.destroy_process_group()


def _cpu_sp_rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rust_neural_network_b200.ops.linear_attention import linear_attention
    from rust_neural_network_b200.parallel.sp import SPContext
    g = torch.Generator().manual_seed(9)
    full = [torch.randn(1, 32 * world, 2, 8, generator=g) for _ in range(3)]
    gy = torch.randn(1, 32 * world, 2, 8, generator=g)
    sp = SPContext(2 * 8 * 16, device="cpu")
    errs = []
    for causal in (True, False):
        ref_in = [t.clone().requires_grad_(True) for t in full]
        ref = linear_attention(*ref_in, scale=0.3, causal=causal, chunk=16)
        ref.backward(gy)
        sl = slice(rank * 32, (rank + 1) * 32)
        loc = [t[:, sl].clone().requires_grad_(True) for t in full]
        got = linear_attention(*loc, scale=0.3, causal=causal, chunk=16, sp=sp)
        got.backward(gy[:, sl])
        errs.append(float((got - ref[:, sl]).abs().max()))
        errs += [float((a.grad - b.grad[:, sl]).abs().max()) for a, b in zip(loc, ref_in)]
    q.put((rank, max(errs)))
    dist.destroy_process_group()


def test_sequence_parallel_linear_attention_three_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cpu_sp_rank, args=(r, 3, 29651, q)) for r in range(3)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(err < 1e-3 for _, err in res), res


def test_tp_baseline_path_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cpu_tp_rank, args=(r, 2, 29641, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, err, scale in res:
        assert err < 2e-2 * scale + 1e-3


def test_tensor_parallel_mlp_autograd_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cpu_tp_mlp_rank, args=(r, 2, 29643, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, errs in res:
        assert max(errs) < 6e-2, errs          # outputs of the baseline path are rounded to bf16; values are O(1..5)


# ------------------------------------------------------------------------------------------------ model level
MODEL_WORKER = str(Path(__file__).resolve().parent / "par_model_worker.py")


def _run_model(nproc, extra, port, timeout=900):
    env = dict(os.environ)
    env.update({"MASTER_ADDR": "127.0.0.1", "OMP_NUM_THREADS": "2", "NCCL_NVLS_ENABLE": "0"})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), MODEL_WORKER] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('{"ranks"')][-1]
    return json.loads(line)["ranks"]


def _check_model(r0, key, grad_tol, loss_tol):
    for k, v in r0["grad_rel_err"].items():
        assert v < grad_tol, (k, v)
    for a, b in zip(r0[key], r0["ref_losses"]):
        assert abs(a - b) < loss_tol, (r0[key], r0["ref_losses"])
    assert r0["ref_losses"][-1] < r0["ref_losses"][0]


def test_tensor_parallel_mamba_lm_two_gloo_ranks():
    """Channel-sharded Mamba blocks on row-sharded activations against the whole model in one process: gradients of
    sharded and of replicated parameters, and the loss over three optimizer steps."""
    r0 = _run_model(2, ["--model", "mamba_tp", "--device", "cpu"], 29661)[0]
    _check_model(r0, "tp_losses", 2e-2, 2e-3)


@pytest.mark.gpu
def test_tensor_parallel_mamba_lm_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r0 = _run_model(2, ["--model", "mamba_tp", "--device", "cuda", "--backend", "fused"], 29662)[0]
    _check_model(r0, "tp_losses", 6e-2, 3e-2)


def test_expert_parallel_moe_lm_two_gloo_ranks():
    """Experts sharded over two ranks (all-to-all baseline path on CPU), shared parameters data-parallel, against the
    same model with every expert local and the whole batch in one process."""
    r0 = _run_model(2, ["--model", "moe_ep", "--device", "cpu"], 29663)[0]
    _check_model(r0, "ep_losses", 3e-2, 3e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("backend,port", [("fused", 29664), ("nccl", 29665)])
def test_expert_parallel_moe_lm_two_gpus(backend, port):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r0 = _run_model(2, ["--model", "moe_ep", "--device", "cuda", "--backend", backend], port)[0]
    _check_model(r0, "ep_losses", 8e-2, 5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("model,key,port", [("mamba_tp", "tp_losses", 29666), ("moe_ep", "ep_losses", 29667)])
def test_parallel_models_eight_gpus(model, key, port):
    """The same two checks over all eight GPUs of a node: 8-way channel sharding, one expert per rank."""
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    r0 = _run_model(8, ["--model", model, "--device", "cuda", "--backend", "fused"], port)[0]
    # the router ("gate") sees 1/8 of the tokens per rank: its load-balance term is taken over the local tokens, the
    # unsharded model's over all of them, and its gradient is a small difference of large sums (0.13 measured)
    gate = r0["grad_rel_err"].pop("gate", 0.0)
    assert gate < 0.25, gate
    _check_model(r0, key, 8e-2, 5e-2)
