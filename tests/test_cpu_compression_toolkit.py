"""compression.py, one test per behaviour of rust-nn src/compression.rs:700-925: weight sharing, CSR matrices, layer
dropping, knowledge transfer, factorised embeddings, per-layer sparsity, progressive shrinking, channel pruning,
the strategy search."""
import pytest
import torch

from rust_neural_network_b200 import compression as C, nn
from rust_neural_network_b200.loss import MSELoss


def _mlp():
    return nn.Sequential().add(nn.Linear(8, 16)).add(nn.ReLU()).add(nn.Linear(16, 4))


def test_weight_sharing_reduces_parameters():
    ws = C.SharedWeights(64, 64, 4)
    assert ws.num_passes == 4 and ws.compression_ratio() > 3.5
    assert tuple(ws.forward(torch.randn(2, 64)).shape) == (2, 64)


def test_sparse_matrix_compression():
    n = 200
    d = torch.eye(n)
    for i in range(n // 5):
        d[i, (i + 1) % n] = 0.5
    sm = C.SparseMatrix.from_dense(d, 0.01)
    assert sm.nnz == n + n // 5 and sm.sparsity() > 0.9 and sm.compression_ratio() > 1.0


def test_sparse_spmm_values():
    sm = C.SparseMatrix.from_dense(torch.tensor([[1.0, 0.0, 0.0], [2.0, 0.0, 3.0]]), 0.01)
    c = sm.spmm(torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0]), 2)
    assert c.reshape(-1).tolist() == pytest.approx([1.0, 2.0, 17.0, 22.0], abs=1e-5)


def test_sparse_to_dense_round_trip():
    d = torch.tensor([[0.5, 0.0, 0.0], [0.3, 0.0, 0.7]])
    assert torch.allclose(C.SparseMatrix.from_dense(d, 0.01).to_dense(), d, atol=1e-5)


def test_layer_dropping_skips_converged_layers():
    ld = C.LayerDropper(3, 0.01)
    x = torch.tensor([1.0, 2.0])
    assert ld.should_skip(0, x, torch.tensor([1.001, 2.001]))
    assert not ld.should_skip(0, x, torch.tensor([2.0, 4.0]))
    assert ld.avg_skip_rate() > 0.0


def test_knowledge_transfer_loss_is_not_negative():
    kt = C.KnowledgeTransfer(nn.Sequential().add(nn.Linear(4, 8)), nn.Sequential().add(nn.Linear(4, 8)), 8, 8)
    assert kt.transfer_loss(torch.randn(2, 4)) >= 0.0


def test_embedding_compression_ratio():
    assert C.CompressedEmbedding.from_table(torch.randn(1000, 256), 32).compression_ratio() > 5.0


def test_embedding_lookup_shapes():
    emb = C.CompressedEmbedding.from_table(torch.randn(100, 64), 16)
    assert tuple(emb.lookup(5).shape) == (1, 64) and tuple(emb.lookup_batch([1, 2, 3]).shape) == (3, 64)


def test_mixed_sparsity_analysis():
    torch.manual_seed(0)
    ms = C.MixedSparsity.analyze(_mlp(), torch.randn(4, 8), torch.randn(4, 4), MSELoss())
    assert ms.layer_sparsity and all(0.0 < s < 1.0 for s in ms.layer_sparsity)


def test_progressive_shrinking_schedule():
    ps = C.ProgressiveShrinking(0.5, 100, 10)
    assert all(ps.step() == 0.0 for _ in range(10))              # warm-up
    r1, r2 = ps.step(), ps.step()
    assert r2 > r1 > 0.0                                          # ramp
    while not ps.is_done():
        ps.step()
    assert abs(ps.current_sparsity - 0.5) < 1e-5


def test_progressive_soft_prune_zeroes_the_smallest():
    ps = C.ProgressiveShrinking(0.5, 100, 10)
    ps.current_sparsity, ps.current_step = 0.3, 50
    t = torch.randn(4, 8)
    pruned = ps.apply_soft_prune(t)
    zeros = pruned == 0
    assert int(zeros.sum()) > 0
    assert float(t[zeros].abs().max()) <= float(t[~zeros].abs().min())


def test_structured_pruning_reduces_channels():
    pruned, kept = C.StructuredPruner.prune_linear(nn.Linear(8, 16), 0.5)
    assert pruned.weight.shape[0] == 8 and len(kept) == 8


def test_structured_pruning_keeps_the_large_channels():
    w = torch.tensor([10.0] * 16 + [0.01] * 16).reshape(4, 8)
    _, kept = C.StructuredPruner.prune_channels(w, 0.5)
    assert sorted(kept) == [0, 1]


def test_automl_finds_a_recipe():
    torch.manual_seed(1)
    recipe = C.automl_search(_mlp(), torch.randn(4, 8), torch.randn(4, 4), MSELoss(), 3.0)
    assert recipe.compression_ratio > 0.0 and recipe.strategies


def test_strategy_size_factors():
    S = C.CompressionStrategy
    assert S.None_().size_factor() == 1.0 and S.Prune(0.5).size_factor() > 1.0 and S.Quantize(8).size_factor() > 3.0
