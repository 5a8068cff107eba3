"""The reference's public functions take its `Tensor` (rust-nn src/activations.rs:6-65, src/loss.rs, src/quantize.rs:85,
src/int8.rs:40, src/fused.rs:60, ...). Here every such entry point accepts the reference-shaped wrapper as well as a
`torch.Tensor`, and answers in kind."""
import torch

import rust_neural_network_b200 as rn
from rust_neural_network_b200.tensor import Tensor as T


def _same(a, b, tol=1e-6):
    a = a.t if isinstance(a, T) else a
    b = b.t if isinstance(b, T) else b
    return torch.allclose(a.float(), b.float(), atol=tol)


def test_activations_take_and_return_the_wrapper():
    x = T.from_vec([1.0, -2.0, 3.0, 0.5], [2, 2])
    for name in ("relu", "sigmoid", "tanh", "gelu", "softmax"):
        f = getattr(rn.activations, name)
        out = f(x)
        assert isinstance(out, T), name
        raw = f(x.t)
        assert isinstance(raw, torch.Tensor) and _same(out, raw), name


def test_losses_and_trainer():
    torch.manual_seed(0)
    lin = rn.Linear(8, 3)
    x, y = T.randn([4, 8]), T.randn([4, 3])
    loss = rn.MSELoss()(lin(x), y)
    assert isinstance(loss, T) and _same(loss, rn.MSELoss()(lin(x.t), y.t))
    loss.backward()
    assert lin.weight.grad is not None
    onehot = T(torch.nn.functional.one_hot(torch.tensor([0, 1, 2, 0]), 3).float())
    assert isinstance(rn.CrossEntropyLoss()(lin(x), onehot), T)
    tr = rn.Trainer(lin, rn.Adam(lin.parameters(), lr=1e-2), rn.MSELoss())
    first = float(T(tr.train_step(x, y)).t)
    for _ in range(20):
        last = float(T(tr.train_step(x, y)).t)
    assert last < first


def test_quantisers_and_compression_take_the_wrapper():
    torch.manual_seed(1)
    x = T.randn([8, 16])
    q = rn.quantize.QuantizedTensor.quantize(x, rn.quantize.QuantFormat.INT8, 0)
    assert q.quantization_error(x) < 0.05 and tuple(q.dequantize().shape) == (8, 16)
    assert rn.int8.Int8Weights.quantize(x).quantization_error(x) < 0.01
    assert rn.ternary.TernaryTensor.quantize(x).compression_ratio() > 5
    assert isinstance(rn.quant.RotorQuant.new(6, 4).quantize(T.randn([5, 6])), T)
    assert rn.compression.SparseMatrix.from_dense(x, 0.5).sparsity() > 0.0
    assert isinstance(rn.distill.softmax_temp(x, 2.0), T)


def test_io_and_tools_take_the_wrapper(tmp_path):
    x = T.from_vec([1.0, 2.0, 3.0, 4.0], [2, 2])
    blob = rn.serialize.serialize([("w", x)])
    (name, back), = rn.deserialize(blob)
    assert name == "w" and _same(back, x)
    s = rn.offload.SsdTensor.write(x, str(tmp_path))
    assert _same(s.load(), x)
    assert "<td" in rn.gui.tensor_heatmap_html(x, 10)
    y = rn.fused.fused_linear(x, T.from_vec([1.0, 0.0, 0.0, 1.0], [2, 2]), None)
    assert isinstance(y, T) and _same(y, x)
    c, _ = rn.gpu_kernels.kernel_matmul(x, x)
    assert isinstance(c, T) and _same(c, x.t @ x.t, 1e-2)
    o = rn.linear_attention.linear_attention_forward(T.randn([1, 4, 2]), T.randn([1, 4, 2]), T.randn([1, 4, 2]), 1, 4, 2, 1.0, 1e-6, False, 0)
    assert isinstance(o, T) and list(o.shape()) == [1, 4, 2]


def test_plain_tensors_pass_through_untouched():
    x = torch.randn(3, 3)
    assert type(rn.activations.relu(x)) is torch.Tensor
    assert type(rn.fused.fused_linear(x, x, None)) is torch.Tensor
    assert type(rn.MSELoss()(x, x)) is torch.Tensor


def test_model_side_methods_take_the_wrapper():
    from rust_neural_network_b200.models.diffusion import DDPM, ScheduleType
    torch.manual_seed(2)
    d = DDPM(3, 16, 100, ScheduleType.Linear)
    xt = d.q_sample(T.from_vec([1.0, 2.0, 3.0], [1, 3]), 0, T.zeros([1, 3]))
    assert isinstance(xt, T) and abs(xt.get([0, 0]) - 1.0) < 0.05
    assert isinstance(d.predict_noise(T.randn([2, 3]), 5), T)
    assert d.train_batch(rn.Adam(d.parameters(), lr=1e-2), T.randn([8, 3])) >= 0.0
    y, loops = rn.LoopedTransformer(4, 8, 2, 16, 2, 3).forward_with_loops(T.randn([1, 3, 4]))
    assert isinstance(y, T) and y.shape() == [1, 3, 2] and loops == 3
    assert isinstance(rn.TreeOfThoughts(4, 2, 2, 1).score(T.randn([2, 4])), T)


def test_the_reference_xor_example_line_by_line():
    """rust-nn examples/xor.rs with `::new` constructors, unit-struct layers and losses, and `Tensor` everywhere."""
    from rust_neural_network_b200 import Adam, Linear, MSELoss, ReLU, Sequential, SimpleDataLoader, Tensor, Trainer
    torch.manual_seed(0)
    inputs = Tensor.from_vec([0.0, 0.0, 0.0, 1.0, 1.0, 0.0, 1.0, 1.0], [4, 2])
    targets = Tensor.from_vec([0.0, 1.0, 1.0, 0.0], [4, 1])
    model = Sequential.new().add(Linear.new(2, 8, True)).add(ReLU).add(Linear.new(8, 1, True))
    trainer = Trainer.new(model, Adam.new(model.parameters(), 0.01), MSELoss)
    losses = [trainer.train_epoch(SimpleDataLoader.new(inputs.clone(), targets.clone(), 4)) for _ in range(200)]
    assert losses[-1] < 0.5 * losses[0]
    out = model.forward(inputs)
    assert isinstance(out, Tensor) and out.shape() == [4, 1]


def test_the_reference_library_usage_loop():
    """rust-nn examples/library_usage.rs: a hand-written loop over a loader built from wrappers yields wrappers."""
    from rust_neural_network_b200 import Adam, Linear, MSELoss, ReLU, Sequential, SimpleDataLoader, Tensor
    torch.manual_seed(1)
    model = Sequential.new().add(Linear.new(10, 32, True)).add(ReLU).add(Linear.new(32, 5, True))
    optimizer = Adam.new(model.parameters(), 0.01)
    loss_fn = MSELoss()
    loader = SimpleDataLoader.new(Tensor.randn([32, 10]), Tensor.randn([32, 5]), 8)
    seen = 0
    for batch_x, batch_y in loader:
        assert isinstance(batch_x, Tensor) and batch_x.shape() == [8, 10]
        optimizer.zero_grad()
        loss = loss_fn.forward(model.forward(batch_x), batch_y)
        loss.backward()
        optimizer.step()
        assert float(loss.data()) > 0.0
        seen += 1
    assert seen == 4
    raw = SimpleDataLoader(torch.randn(5, 2), torch.randn(5, 1), 2)          # torch tensors in, torch tensors out
    assert all(type(x) is torch.Tensor for x, _ in raw) and len(raw) == 3


def test_reference_field_names_read_this_packages_fields():
    from rust_neural_network_b200 import nn, position
    from rust_neural_network_b200.models import looped_transformer as LT
    assert nn.LayerNorm(4).num_features == 4 and nn.BatchNorm1D(6).num_features == 6
    csa = nn.CSA(8, 2)
    assert csa.group_size == 2 and csa.compression_layer is csa.compression
    assert position.RoPE.new(8, 16).scale == 1.0 and position.RoPE.yarn(8, 16, 10000.0, 4.0).scale == 4.0
    mha = LT.MultiHeadAttention(8, 2)
    assert (mha.num_heads, mha.head_dim) == (2, 4)
    blk = LT.TransformerBlock(8, 2, 16)
    assert (blk.d_model, blk.ff_dim) == (8, 16) and blk.ff.parameters()[0] is blk.ff1.weight
    ln = nn.LayerNorm(4)
    ln.num_features = 7                                              # an alias never blocks an assignment
    assert ln.num_features == 7 and ln.n == 4


def test_expert_views_compose_to_the_layer():
    """`moe.experts[e]` is expert e on its own: with every expert selected, the layer equals the gate-weighted sum."""
    torch.manual_seed(3)
    moe = rn.NormalMoE(8, 16, 4, top_k=4)
    x = torch.randn(5, 8)
    w = torch.softmax(moe.gate(x).detach().float(), -1)
    want = sum(w[:, e:e + 1] * moe.experts[e](x).float() for e in range(4))
    assert len(moe.experts) == 4 and torch.allclose(moe(x).detach().float(), want.detach(), atol=1e-4)


def test_compat_layer_rules():
    from rust_neural_network_b200._compat import accept_wrapped, alias_fields, rewrap, unwrap

    @accept_wrapped
    def f(a, pairs=(), scale=1.0, *, extra=None):
        total = a * scale
        for _, t in pairs:
            total = total + t
        return (total + extra, [total]) if extra is not None else total

    x, y = T.from_vec([1.0, 2.0], [2]), T.from_vec([10.0, 20.0], [2])
    assert type(f(x.t)) is torch.Tensor                                   # nothing wrapped: untouched
    out = f(x, [("w", y)], 2.0)                                           # wrappers inside (name, tensor) pairs count
    assert isinstance(out, T) and out.data().tolist() == [12.0, 24.0]
    a, (b,) = f(x.t, extra=y)                                             # a wrapped keyword argument, a nested result
    assert isinstance(a, T) and isinstance(b, T) and a.data().tolist() == [11.0, 22.0]
    assert accept_wrapped(f) is f                                         # wrapping twice is a no-op
    p = torch.nn.Parameter(torch.zeros(2))
    assert rewrap(p) is p and unwrap([x, (y, 3)])[1][1] == 3              # parameters stay parameters; other values pass through

    class Box:
        def __init__(self):
            self.n = 5
    alias_fields(Box, size="n", double=lambda self: 2 * self.n)
    bx = Box()
    assert (bx.size, bx.double) == (5, 10)
    bx.size = 9                                                            # an instance attribute wins
    assert bx.size == 9 and bx.n == 5


def test_gathered_rows_are_kept_without_a_copy_off_the_fused_path():
    """`TPContext.keep_gathered` on the NCCL / gloo path: the gathered tensor is already private, no copy, no event."""
    from rust_neural_network_b200.parallel.tp import TPContext
    ctx = TPContext.__new__(TPContext)
    ctx.backend = "nccl"
    xg = torch.randn(4, 3)
    kept, done = ctx.keep_gathered(xg)
    assert kept is xg and done is None
    ctx.join_copy()                                                        # nothing outstanding: a no-op
