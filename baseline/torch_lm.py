"""Library baseline for the headline benchmark: the same looped-transformer LM written with stock PyTorch
modules only (cuBLAS GEMMs through `nn.Linear`, `scaled_dot_product_attention`, `nn.LayerNorm`,
`F.cross_entropy`, the fused `torch.optim.Adam`, `DistributedDataParallel` over NCCL). None of this
package's kernels are on this path; it exists so that `bench.py --impl torch` measures the number the
hand-written sm_100a path has to beat on the same box, same shapes, same precision policy (bf16 compute
through autocast, fp32 master weights and optimizer state).

The architecture mirrors `rust_neural_network_b200.models.lm.LoopedTransformerLM`: token + learned position
embeddings, a shared block of pre-norm layers applied `loops` times with a per-loop time embedding added to
the stream, final LayerNorm, LM head with bias, mean token cross-entropy.
"""
from __future__ import annotations

import torch
import torch.nn as tnn
import torch.nn.functional as TF


class Layer(tnn.Module):
    def __init__(self, d, heads, ff):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = tnn.LayerNorm(d), tnn.LayerNorm(d)
        self.qkv, self.o = tnn.Linear(d, 3 * d), tnn.Linear(d, d)
        self.ff1, self.ff2 = tnn.Linear(d, ff), tnn.Linear(ff, d)

    def forward(self, x, causal):
        B, S, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = TF.scaled_dot_product_attention(q, k, v, is_causal=causal)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, d))
        return x + self.ff2(TF.gelu(self.ff1(self.ln2(x))))


class TorchLoopedLM(tnn.Module):
    def __init__(self, vocab, d_model, heads, ff_dim, layers_per_block, loops, max_seq, causal=True, init_std=0.02):
        super().__init__()
        self.loops, self.causal = loops, causal
        self.tok, self.pos = tnn.Embedding(vocab, d_model), tnn.Embedding(max_seq, d_model)
        self.block = tnn.ModuleList(Layer(d_model, heads, ff_dim) for _ in range(layers_per_block))
        self.time = tnn.Embedding(loops, d_model)
        self.ln_final = tnn.LayerNorm(d_model)
        self.lm_head = tnn.Linear(d_model, vocab)
        for m in self.modules():
            if isinstance(m, (tnn.Linear, tnn.Embedding)):
                tnn.init.normal_(m.weight, std=init_std)
            if isinstance(m, tnn.Linear):
                tnn.init.zeros_(m.bias)

    def forward(self, ids, labels):
        B, S = ids.shape
        h = self.tok(ids) + self.pos(torch.arange(S, device=ids.device))
        for t in range(self.loops):
            h = h + self.time.weight[t]
            for layer in self.block:
                h = layer(h, self.causal)
        logits = self.lm_head(self.ln_final(h))
        return TF.cross_entropy(logits.float().view(B * S, -1), labels.view(-1))


class TorchStep:
    """One training step (forward, backward, Adam) on static device buffers, optionally replayed as a CUDA graph."""

    def __init__(self, model, batch, seq, device, world, lr=1e-3, graph=True):
        self.model = model
        self.net = model
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel
            self.net = DistributedDataParallel(model, device_ids=[device.index], gradient_as_bucket_view=True)
            graph = False                      # stock DDP reducers are not captured here
        self.opt = torch.optim.Adam(model.parameters(), lr=lr, fused=not graph, capturable=graph)
        self.ids = torch.zeros(batch, seq, dtype=torch.long, device=device)
        self.labels = torch.zeros(batch, seq, dtype=torch.long, device=device)
        self.loss = torch.zeros((), device=device)
        self.graph = None
        self.want_graph = graph

    def _eager(self):
        self.opt.zero_grad(set_to_none=False)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.net(self.ids, self.labels)
        loss.backward()
        self.opt.step()
        self.loss.copy_(loss.detach())

    def warmup(self, n):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(max(n, 3)):
                self._eager()
        torch.cuda.current_stream().wait_stream(s)
        if self.want_graph:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._eager()

    def step_device(self, ids, labels):
        self.ids.copy_(ids, non_blocking=True)
        self.labels.copy_(labels, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._eager()
        return self.loss


def flops_per_token(cfg):
    d, ff, L, S, V = cfg["d_model"], cfg["ff_dim"], cfg["layers_per_block"] * cfg["loops"], cfg["seq_len"], cfg["vocab"]
    per_layer = 2 * (4 * d * d + 2 * d * ff) + 2 * 2 * S * d / 2          # projections + causal attention
    return 3 * (L * per_layer + 2 * d * V)


__all__ = ["TorchLoopedLM", "TorchStep", "flops_per_token"]
