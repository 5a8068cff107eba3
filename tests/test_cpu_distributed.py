"""distributed.py host runtime, one test per behaviour of rust-nn src/distributed.rs:530-735: the simulated ring
all-reduce (the oracle of the fused data-parallel kernel), gradient averaging, data sharding, learning-rate scaling,
message framing and its rejections, gradient clipping, flatten / unflatten, the standalone worker."""
import torch

from rust_neural_network_b200 import distributed as D
from rust_neural_network_b200 import nn


def test_ring_all_reduce_2_workers():
    w = [[1.0] * 8, [2.0] * 8]
    D.ring_all_reduce_all(w, 2)
    assert all(abs(v - 3.0) < 1e-5 for row in w for v in row)


def test_ring_all_reduce_4_workers():
    w = [[r + 1.0] * 12 for r in range(4)]
    D.ring_all_reduce_all(w, 4)
    assert all(abs(v - 10.0) < 1e-4 for row in w for v in row)


def test_ring_all_reduce_uneven_chunks():
    w = [[float(r * 10 + i) for i in range(7)] for r in range(3)]          # 7 elements over 3 workers: ragged chunks
    want = [sum(r * 10 + i for r in range(3)) for i in range(7)]
    D.ring_all_reduce_all(w, 3)
    for row in w:
        assert all(abs(a - b) < 1e-4 for a, b in zip(row, want))


def test_ring_all_reduce_single_worker_is_a_no_op():
    w = [[1.0, 2.0, 3.0]]
    D.ring_all_reduce_all(w, 1)
    assert w[0] == [1.0, 2.0, 3.0]


def test_average_gradients():
    data = [10.0, 20.0, 30.0]
    D.average_gradients(data, 4)
    assert [round(v, 6) for v in data] == [2.5, 5.0, 7.5]


def test_data_sharding_has_no_overlap():
    ranges = [D.DistributedConfig.new(r, 4).shard_range(100) for r in range(4)]
    assert ranges == [(0, 25), (25, 50), (50, 75), (75, 100)]


def test_data_sharding_with_remainder():
    (s0, e0), (s1, e1), (s2, e2) = (D.DistributedConfig.new(r, 3).shard_range(100) for r in range(3))
    assert (e0 - s0, e1 - s1, e2 - s2) == (34, 33, 33)                      # rank 0 takes the extra sample
    assert s0 == 0 and s1 == e0 and s2 == e1 and e2 == 100


def test_lr_scaling():
    assert abs(D.DistributedConfig.new(0, 8).effective_lr(0.001) - 0.008) < 1e-9
    cfg = D.DistributedConfig.new(0, 8)
    cfg.scale_lr = False
    assert abs(cfg.effective_lr(0.001) - 0.001) < 1e-9


def test_local_batch_size():
    cfg = D.DistributedConfig.new(0, 4)
    assert cfg.local_batch_size(128) == 32 and cfg.local_batch_size(4) == 1 and cfg.local_batch_size(2) == 1


def test_message_round_trip():
    raw = D.Message.gradient_chunk([1.0, 2.0, 3.0]).serialize()
    assert len(raw) == 1 + 4 + 12
    m = D.Message.deserialize(raw)
    assert m.msg_type == D.MessageType.GradientChunk and m.as_floats() == [1.0, 2.0, 3.0]


def test_message_barrier_is_five_bytes():
    raw = D.Message.barrier().serialize()
    assert len(raw) == 5
    m = D.Message.deserialize(raw)
    assert m.msg_type == D.MessageType.Barrier and len(m.payload) == 0


def test_message_with_an_unknown_type_is_rejected():
    assert D.Message.deserialize(bytes([99, 0, 0, 0, 0])) is None


def test_truncated_message_is_rejected():
    raw = D.Message.gradient_chunk([1.0, 2.0]).serialize()
    assert D.Message.deserialize(raw[:-2]) is None
    assert D.Message.deserialize(raw[:3]) is None


def test_gradient_clipping():
    model = nn.Sequential().add(nn.Linear(4, 4))
    params = model.parameters()
    for p in params:
        p.grad = torch.full_like(p, 100.0)
    before = D.clip_gradients(params, 1.0)
    assert before > 100.0
    norm = sum(float((p.grad ** 2).sum()) for p in params) ** 0.5
    assert norm <= 1.01
    small = [torch.zeros(3, requires_grad=True)]
    small[0].grad = torch.full((3,), 0.1)
    D.clip_gradients(small, 1.0)
    assert torch.allclose(small[0].grad, torch.full((3,), 0.1))             # below the threshold: untouched


def test_flatten_unflatten_round_trip():
    t1, t2 = torch.zeros(2, 2, requires_grad=True), torch.zeros(2, requires_grad=True)
    t1.grad, t2.grad = torch.ones(2, 2), torch.full((2,), 2.0)
    flat = D.flatten_gradients([t1, t2])
    assert flat.numel() == 6
    D.unflatten_gradients([t1, t2], flat * 3.0)
    assert float(t1.grad[0, 0]) == 3.0 and float(t2.grad[0]) == 6.0


def test_standalone_worker():
    w = D.DistributedWorker.standalone(2, 4)
    assert w.config.rank == 2 and w.config.world_size == 4
