"""The three language-model families on a toy problem: looped transformer, Mamba, FineGrainedMoE transformer. Each trains
for a few steps on random tokens through `Trainer` and must reduce its loss. bf16 compute on a GPU, fp32 on a CPU.

    python examples/language_models.py
"""
import _common
import torch

from rust_neural_network_b200 import Adam, Trainer
from rust_neural_network_b200.models.lm import LoopedTransformerLM
from rust_neural_network_b200.models.mamba import MambaLM
from rust_neural_network_b200.models.moe import MoETransformerLM

dev = _common.device()
dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
V, S, B = 128, 128, 4
torch.manual_seed(0)
ids = torch.randint(0, V, (B, S))
labels = torch.roll(ids, -1, dims=1)
models = {
    "looped transformer": LoopedTransformerLM(V, 128, 2, 256, layers_per_block=2, loops=2, max_seq=S),
    "mamba": MambaLM(V, 128, 2, d_state=16, dt_rank=8),
    "moe transformer": MoETransformerLM(V, 128, 2, 2, num_experts=8, top_k=2, num_shared=1, expert_hidden=128, max_seq=S),
}
for name, model in models.items():
    model.to_device(dev, dt)
    tr = Trainer(model, Adam(model.parameters(), lr=3e-3))
    losses = [float(tr.train_step(ids, labels)) for _ in range(20)]
    print(f"{name:20s} params {model.num_parameters():8d}  loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    assert losses[-1] < losses[0]
