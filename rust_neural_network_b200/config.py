"""Named presets for the benchmark configurations this framework is measured on, as dataclasses in the
style of the reference's config structs (`DistributedConfig`, `FastTrainConfig`, ... rust-nn
src/distributed.rs:202-263, src/finetune.rs:209-279), plus the environment namespace:

  RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT   process-group rendezvous (RUST_NN_RANK / RUST_NN_WORLD_SIZE /
                                                  RUST_NN_MASTER are accepted as aliases, see `distributed.init_from_env`)
  B200NN_DP_MULTIMEM=1                            fused data-parallel step uses multimem.ld_reduce / multimem.st
  HF_TOKEN, HUGGING_FACE_HUB_TOKEN, KAGGLE_USERNAME, KAGGLE_KEY, HOME    as the reference (src/data.rs:854-858)
"""
from __future__ import annotations

import dataclasses
from typing import Dict

import torch


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    """784 -> 256 -> ReLU -> 128 -> ReLU -> 10, Kaiming-uniform init, cross-entropy, Adam 1e-3, fp32, batch 32, 100 steps."""
    dims: tuple = (784, 256, 128, 10)
    batch: int = 32
    lr: float = 1e-3
    steps: int = 100
    dtype: str = "float32"


@dataclasses.dataclass(frozen=True)
class LoopedLmConfig:
    """Looped transformer LM: 4 pre-norm layers looped 6 times, d 512, 8 heads x 64, GELU FFN 2048, causal flash attention."""
    vocab: int = 32000
    d_model: int = 512
    heads: int = 8
    ff_dim: int = 2048
    layers_per_block: int = 4
    loops: int = 6
    seq_len: int = 1024
    global_batch: int = 64
    init_std: float = 0.02
    parallelism: str = "dp"


@dataclasses.dataclass(frozen=True)
class MoeLmConfig:
    """FineGrainedMoE transformer: d 1024, 16 layers, 16 heads, 64 routed experts top-6 + 2 shared, expert hidden 512 SiLU."""
    vocab: int = 32000
    d_model: int = 1024
    layers: int = 16
    heads: int = 16
    num_experts: int = 64
    top_k: int = 6
    num_shared: int = 2
    expert_hidden: int = 512
    seq_len: int = 2048
    batch_per_gpu: int = 32
    parallelism: str = "ep"


@dataclasses.dataclass(frozen=True)
class MambaLmConfig:
    """Mamba (S6) LM: d 2048, 24 layers, d_state 16, d_conv 4, expand 2, dt_rank 128, seq 4096, batch 8 per GPU."""
    vocab: int = 32000
    d_model: int = 2048
    layers: int = 24
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    dt_rank: int = 128
    seq_len: int = 4096
    batch_per_gpu: int = 8
    parallelism: str = "tp"
    recompute_scan: bool = False     # rebuild the scan's state checkpoints in the backward instead of keeping them per layer


@dataclasses.dataclass(frozen=True)
class AttentionSweepConfig:
    """Forward + backward of causal linear attention (ELU+1, ReLU^2) against flash attention."""
    batch: int = 8
    heads: int = 16
    head_dims: tuple = (64, 128)
    seq_lens: tuple = (1024, 4096, 16384, 65536)
    sequence_parallel_from: int = 65536


PRESETS: Dict[str, object] = {
    "mlp": MlpConfig(), "looped_lm": LoopedLmConfig(), "moe_lm": MoeLmConfig(), "mamba_lm": MambaLmConfig(), "attention_sweep": AttentionSweepConfig(),
}


def build_model(name: str, device="cuda", tp=None, ep_group=None, ep_backend: str = "fused", **overrides):
    """Instantiates the model of a preset (bf16 compute on CUDA, fp32 on CPU). `overrides` replace preset fields.
    `tp` (a `parallel.tp.TPContext`) builds the tensor-parallel Mamba LM, `ep_group` the expert-parallel MoE LM."""
    cfg = dataclasses.replace(PRESETS[name], **overrides)
    dev = torch.device(device)
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    if name == "mlp":
        from . import nn
        m = nn.Sequential()
        d = cfg.dims
        for i in range(len(d) - 1):
            m.add(nn.Linear(d[i], d[i + 1], init=nn.kaiming_uniform))
            if i + 2 < len(d):
                m.add(nn.ReLU())
        return m.to_device(dev, torch.float32), cfg
    if name == "looped_lm":
        from .models.lm import LoopedTransformerLM
        m = LoopedTransformerLM(cfg.vocab, cfg.d_model, cfg.heads, cfg.ff_dim, cfg.layers_per_block, cfg.loops, cfg.seq_len, causal=True)
        return m.to_device(dev, dt), cfg
    if name == "moe_lm":
        from .models.moe import MoETransformerLM
        m = MoETransformerLM(cfg.vocab, cfg.d_model, cfg.layers, cfg.heads, cfg.num_experts, cfg.top_k, cfg.num_shared, cfg.expert_hidden, cfg.seq_len,
                             ep_group=ep_group, ep_backend=ep_backend)
        return m.to_device(dev, dt), cfg
    if name == "mamba_lm":
        from .models.mamba import MambaLM
        m = MambaLM(cfg.vocab, cfg.d_model, cfg.layers, d_state=cfg.d_state, d_conv=cfg.d_conv, expand=cfg.expand, dt_rank=cfg.dt_rank, tp=tp, recompute_scan=cfg.recompute_scan)
        return m.to_device(dev, dt), cfg
    raise KeyError(name)
