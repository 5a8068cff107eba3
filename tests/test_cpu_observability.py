"""Metrics logger, roofline calculator, kernel report, and configuration presets."""
import json

import torch

from rust_neural_network_b200 import config
from rust_neural_network_b200.utils import metrics


def test_metrics_logger_and_roofline(tmp_path):
    p = tmp_path / "m" / "run.jsonl"
    log = metrics.MetricsLogger(str(p))
    log.log(1, loss=torch.tensor(2.5), tokens_per_s=1e5, hist=torch.tensor([1.0, 2.0]))
    log.log(2, loss=1.5)
    lines = [json.loads(l) for l in p.read_text().splitlines()]
    assert len(lines) == 2 and lines[0]["loss"] == 2.5 and lines[0]["hist"] == [1.0, 2.0] and lines[1]["step"] == 2
    assert log.losses() == [2.5, 1.5]
    pk = metrics.measured_peaks()
    assert pk["kind"] in ("of measured", "of fallback") and pk["hbm_gbs"] > 1000 and pk["bf16_tflops"] > 100
    r = metrics.roofline(1.0, flops=pk["bf16_tflops"] * 1e9 * 0.5, bytes_moved=pk["hbm_gbs"] * 1e6 * 0.25)
    assert abs(r["frac_of_bf16_peak"] - 0.5) < 1e-6 and abs(r["frac_of_hbm_peak"] - 0.25) < 1e-6 and abs(r["frac_of_roofline"] - 0.5) < 1e-6
    link = metrics.roofline(1.0, flops=1e9, nvlink_bytes=770e6)
    assert abs(link["roofline_ms"] - 1.0) < 1e-6                       # NVLink-bound target: 770 MB at 770 GB/s
    rep = metrics.kernel_report()
    assert rep["arch"] == "sm_100a" and rep["cuda_library"].endswith("libb200nn_cuda.so") and rep["host_library_present"]


def test_config_presets():
    assert set(config.PRESETS) == {"mlp", "looped_lm", "moe_lm", "mamba_lm", "attention_sweep"}
    lm = config.PRESETS["looped_lm"]
    assert (lm.d_model, lm.heads, lm.layers_per_block, lm.loops, lm.ff_dim, lm.vocab, lm.seq_len, lm.global_batch) == (512, 8, 4, 6, 2048, 32000, 1024, 64)
    moe = config.PRESETS["moe_lm"]
    assert (moe.num_experts, moe.top_k, moe.num_shared, moe.expert_hidden) == (64, 6, 2, 512)
    m, cfg = config.build_model("mlp", device="cpu")
    assert [tuple(p.shape) for p in m.parameters() if p.dim() == 2] == [(256, 784), (128, 256), (10, 128)]
    small, cfg2 = config.build_model("looped_lm", device="cpu", vocab=64, d_model=32, heads=2, ff_dim=64, layers_per_block=1, loops=2, seq_len=16)
    ids = torch.randint(0, 64, (2, 16))
    assert tuple(small(ids).shape) == (2, 16, 64) and cfg2.loops == 2
    mm, _ = config.build_model("mamba_lm", device="cpu", vocab=64, d_model=32, layers=2, dt_rank=4, seq_len=16)
    assert tuple(mm(ids).shape) == (2, 16, 64)
    mo, _ = config.build_model("moe_lm", device="cpu", vocab=64, d_model=32, layers=1, heads=2, num_experts=4, top_k=2, num_shared=1, expert_hidden=16, seq_len=16)
    assert tuple(mo(ids).shape) == (2, 16, 64)


def test_trainer_and_fast_trainer_write_metrics_lines(tmp_path):
    """The JSONL logger is fed by the training loops themselves (one record per logged step)."""
    import json

    import torch

    from rust_neural_network_b200 import nn
    from rust_neural_network_b200.finetune import FastTrainConfig, FastTrainer
    from rust_neural_network_b200.loss import MSELoss
    from rust_neural_network_b200.optim import Adam
    from rust_neural_network_b200.train import SimpleDataLoader, Trainer
    from rust_neural_network_b200.utils.metrics import MetricsLogger
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(4, 8)).add(nn.ReLU()).add(nn.Linear(8, 1))
    x, y = torch.randn(16, 4), torch.randn(16, 1)
    log = MetricsLogger(str(tmp_path / "train.jsonl"))
    tr = Trainer(model, Adam(model.parameters(), lr=1e-2), MSELoss("mean"), logger=log, log_every=2)
    tr.train_epoch(SimpleDataLoader(x, y, 4))
    lines = [json.loads(l) for l in (tmp_path / "train.jsonl").read_text().splitlines()]
    assert [r["step"] for r in lines] == [2, 4] and all("loss" in r for r in lines)
    log2 = MetricsLogger(str(tmp_path / "fast.jsonl"))
    cfg = FastTrainConfig()
    cfg.epochs, cfg.micro_batch_size, cfg.log_every = 2, 4, 1
    FastTrainer(model, cfg, logger=log2).fit(SimpleDataLoader(x, y, 4), Adam(model.parameters(), lr=1e-2), MSELoss("mean"))
    assert len(log2.records) >= 2 and all("lr" in r for r in log2.records)


def test_nvtx_ranges_are_free_without_a_gpu_and_profile_exports_a_trace(tmp_path):
    import json

    import torch

    from rust_neural_network_b200.ops.gemm import gemm
    from rust_neural_network_b200.utils import metrics
    with metrics.nvtx_range("anything"):
        pass
    with metrics.profile_to(str(tmp_path / "trace.json")):
        gemm(torch.randn(8, 8), torch.randn(8, 8))
    assert "traceEvents" in json.loads((tmp_path / "trace.json").read_text())
