"""Data-parallel optimizer tests. CPU: two gloo ranks run the all-reduce path and must reproduce the
single-process result (Adam, Adam + global-norm clipping, Muon, checkpoint written at world 2 and reloaded at
world 1). GPU (needs >= 2 devices): the fused reduce-scatter + optimizer + all-gather kernels over peer
memory must do the same, keep every value the forward consumes bit-identical on all ranks, and survive a
CUDA-graph replay with one rank delayed."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

WORKER = str(Path(__file__).resolve().parent / "ddp_worker.py")


def _run(nproc, extra, port, timeout=600, env_extra=None):
    env = dict(os.environ)
    env.update({"MASTER_ADDR": "127.0.0.1", "OMP_NUM_THREADS": "2"})
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('{"ranks"')][-1]
    return json.loads(line)["ranks"]


# fp32 on CPU: the two-rank result differs from the single-process one only by summation order
@pytest.mark.parametrize("extra,port", [([], 29611), (["--clip", "0.5"], 29612), (["--opt", "muon"], 29613)])
def test_two_gloo_ranks_match_single_process(extra, port):
    ranks = _run(2, ["--device", "cpu", "--mode", "nccl", "--steps", "2"] + extra, port)
    r0 = ranks[0]
    assert r0["rel_update_size"] > 1e-4
    assert r0["err_over_update"] < 0.05
    assert r0["worst_replicated_param_err_over_update"] < 0.05
    if "--clip" in extra:
        assert r0["norm"] > 0.5                       # the threshold was active: the oracle match above proves the coefficient


def test_checkpoint_written_at_world2_reloads_at_world1(tmp_path):
    """save_checkpoint at world 2, load into a single-process model + optimizer: weights and Adam moments equal the
    single-process run's (the sidecar is keyed per parameter, so the optimizers' different flat layouts do not matter)."""
    _run(2, ["--device", "cpu", "--mode", "nccl", "--steps", "2", "--ckpt", str(tmp_path)], 29614)
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    import ddp_worker as W
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.serialize import load_checkpoint
    dev = torch.device("cpu")
    a, b = W.build(dev, torch.float32), W.build(dev, torch.float32)
    oa, ob = Adam(a.parameters(), lr=1e-3), Adam(b.parameters(), lr=1e-3)
    load_checkpoint(str(tmp_path / "dp.rnnb"), a, oa)
    load_checkpoint(str(tmp_path / "single.rnnb"), b, ob)
    assert float(oa.step_t) == float(ob.step_t) == 2.0
    for name, x, y in (("m", oa.m, ob.m), ("v", oa.v, ob.v), ("w", oa.flat.master, ob.flat.master)):
        assert float(y.abs().max()) > 0
        assert float((x - y).abs().max()) <= 1e-3 * float(y.abs().max()) + 1e-12, name


def _gpu_case(extra, port):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    return _run(2, ["--device", "cuda", "--steps", "3"] + extra, port, env_extra={"NCCL_NVLS_ENABLE": "0"})


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_two_gpu_ranks_match_single_process(mode):
    ranks = _gpu_case(["--mode", mode], 29621 if mode == "nccl" else 29622)
    r0 = ranks[0]
    assert r0["mode"] == mode
    assert r0["rel_update_size"] > 1e-4
    # bf16 forward/backward on different batch splits: agreement well inside the size of the update itself
    assert r0["err_over_update"] < 0.25
    # biases and LayerNorm parameters are updated in fp32 from the same averaged gradient on every rank
    assert r0["replicated_err_over_update"] < 0.25
    assert r0["worst_replicated_param_err_over_update"] < 0.5
    assert r0["shadow_err"] == 0.0
    if mode == "fused":
        assert r0["n_replicated"] > 0
        assert all(r["shadow_mismatch_vs_rank0"] == 0.0 for r in ranks)
        assert all(r["replicated_master_mismatch_vs_rank0"] == 0.0 for r in ranks)


@pytest.mark.gpu
@pytest.mark.parametrize("extra,port", [(["--clip", "0.5"], 29623), (["--opt", "muon"], 29624), (["--groups", "1"], 29625),
                                        (["--groups", "1", "--clip", "0.5"], 29626)])
def test_two_gpu_fused_variants(extra, port):
    """Two-pass launches (clipping by the norm of the averaged gradient, Muon's per-tensor RMS) and bucketed launches
    overlapped with backward."""
    ranks = _gpu_case(["--mode", "fused"] + extra, port)
    r0 = ranks[0]
    assert r0["err_over_update"] < 0.25
    assert r0["worst_replicated_param_err_over_update"] < 0.5
    assert all(r["shadow_mismatch_vs_rank0"] == 0.0 for r in ranks)
    assert all(r["replicated_master_mismatch_vs_rank0"] == 0.0 for r in ranks)
    if "--groups" in extra:
        assert r0["buckets"] >= 2
    if "--clip" in extra:
        assert r0["norm"] > 0.5
    # guard bands around every symmetric buffer are intact on every rank, and the check notices a changed byte
    assert all(r["canaries_checked"] >= 3 and r["canary_detects"] for r in ranks)


@pytest.mark.gpu
def test_two_gpu_graph_replay_with_a_delayed_rank():
    """The captured step (Trainer snapshots and restores the optimizer state around its warm-up, which rewinds the Adam
    step) must still make every rank wait for its peers: rank 1 sleeps before each replay."""
    ranks = _gpu_case(["--mode", "fused", "--graph", "1"], 29627)
    assert ranks[0]["graph_vs_eager_over_update"] < 0.05
    assert all(r["shadow_mismatch_vs_rank0"] == 0.0 for r in ranks)


@pytest.mark.gpu
def test_two_gpu_fused_checkpoint_gathers_moments(tmp_path):
    _gpu_case(["--mode", "fused", "--ckpt", str(tmp_path)], 29628)
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    import ddp_worker as W
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.serialize import load_checkpoint
    dev = torch.device("cuda", 0)
    a, b = W.build(dev, torch.bfloat16), W.build(dev, torch.bfloat16)
    oa, ob = Adam(a.parameters(), lr=1e-3), Adam(b.parameters(), lr=1e-3)
    load_checkpoint(str(tmp_path / "dp.rnnb"), a, oa)
    load_checkpoint(str(tmp_path / "single.rnnb"), b, ob)
    for name, x, y in (("m", oa.m, ob.m), ("v", oa.v, ob.v)):
        # every slice of the moments is present (none left at zero) and close to the single-process ones
        rel = float((x - y).norm() / y.norm())
        assert rel < 0.25, (name, rel)
