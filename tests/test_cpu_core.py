"""CPU tests of the framework surface (no GPU needed): tensor facade, modules, losses, optimizers,
checkpoints (golden bytes of the rnnb v1 format), positional encodings, the deterministic generator.
Where a kernel exists the CPU path is the fp32 PyTorch reference of the same op, so these tests
also pin the oracles the GPU tests compare against."""
import math
import struct

import pytest
import torch

from rust_neural_network_b200 import nn, serialize
from rust_neural_network_b200.error import SerializationError, ShapeMismatch, checked_add, checked_matmul, checked_reshape
from rust_neural_network_b200.loss import BCELoss, BCEWithLogitsLoss, CrossEntropyLoss, HuberLoss, L1Loss, MSELoss
from rust_neural_network_b200.models.looped_transformer import AttentionKind, LoopedTransformer, MultiHeadAttention, Transformer, TransformerBlock
from rust_neural_network_b200.models.mamba import HybridMamba, Mamba, MambaBlock, MambaLM
from rust_neural_network_b200.optim import SGD, Adam, Muon, RMSprop
from rust_neural_network_b200.position import AlibiBias, CARoPE, LearnedPE, RoPE, SinusoidalPE
from rust_neural_network_b200.tensor import Tensor
from rust_neural_network_b200.train import SimpleDataLoader, Trainer
from rust_neural_network_b200.utils.lcg import lcg_tensor, lcg_values


# ----------------------------------------------------------------------------- generator
def test_lcg_matches_scalar_recurrence():
    x, ref = 7, []
    for _ in range(100):
        x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
        ref.append((x >> 8) / 16777216.0 - 0.5)
    assert torch.allclose(torch.tensor(lcg_values(100, 7)), torch.tensor(ref, dtype=torch.float32))
    assert lcg_tensor((3, 4), 1).shape == (3, 4)


# ----------------------------------------------------------------------------- tensor facade
def test_tensor_api_semantics():
    t = Tensor.from_vec([1, 2, 3, 4, 5, 6], [2, 3])
    assert t.shape() == [2, 3] and t.ndim() == 2 and t.len() == 6 and not t.is_empty()
    assert t.transpose().shape() == [3, 2]
    assert Tensor.zeros([2, 3, 4]).transpose().shape() == [4, 3, 2]      # reverses ALL axes
    assert t.sum().shape() == [] and t.mean() == 3.5 and t.max() == 6.0 and t.min() == 1.0
    assert t.argmax() == 5 and t.get_idx(4) == 5.0 and t.get([1, 0]) == 4.0
    with pytest.raises(ShapeMismatch):
        Tensor.from_vec([1, 2, 3], [2, 2])
    assert Tensor.he([4, 8]).requires_grad() and Tensor.xavier([4, 8]).requires_grad()
    assert not Tensor.randn([2, 2]).requires_grad()
    a = Tensor.new([[1.0, 2.0], [3.0, 4.0]], True)
    b = Tensor.new([[0.5, -1.0], [2.0, 1.0]], True)
    c = (a * b + a - b).matmul(a).relu().sum()
    c.backward()
    ar = a.t.detach().clone().requires_grad_(True); br = b.t.detach().clone().requires_grad_(True)
    torch.relu((ar * br + ar - br) @ ar).sum().backward()
    assert torch.allclose(a.grad(), ar.grad) and torch.allclose(b.grad(), br.grad)
    assert t.clamp(2, 4).flat_data() == [2, 2, 3, 4, 4, 4]
    with pytest.raises(ShapeMismatch):
        a.matmul(Tensor.zeros([3, 2]))


def test_checked_ops():
    a, b = Tensor.ones([2, 3]), Tensor.ones([3, 4])
    assert checked_matmul(a, b).shape() == [2, 4]
    with pytest.raises(ShapeMismatch):
        checked_matmul(a, a)
    with pytest.raises(ShapeMismatch):
        checked_reshape(a, [4, 2])
    with pytest.raises(ShapeMismatch):
        checked_add(a, b)
    assert checked_add(a, Tensor.ones([3])).shape() == [2, 3]


# ----------------------------------------------------------------------------- modules / losses
def test_linear_layernorm_batchnorm_against_torch():
    torch.manual_seed(0)
    lin = nn.Linear(5, 3)
    assert lin.weight.shape == (3, 5) and float(lin.bias.abs().sum()) == 0.0
    x = torch.randn(4, 5, requires_grad=True)
    y = lin(x)
    assert torch.allclose(y, x @ lin.weight.t() + lin.bias, atol=1e-6)
    ln = nn.LayerNorm(5)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (5,), ln.gamma, ln.beta, 1e-5), atol=1e-5)
    bn = nn.BatchNorm1D(5)
    ref = torch.nn.BatchNorm1d(5)
    yb = bn(x); yr = ref(x)
    assert torch.allclose(yb, yr, atol=1e-5)
    assert torch.allclose(bn.buf_running_mean, ref.running_mean, atol=1e-6)
    bn.eval(); ref.eval()
    assert torch.allclose(bn(x), ref(x), atol=1e-5)
    with pytest.raises(ValueError):
        bn(torch.randn(2, 3, 5))


def test_activations_are_differentiable_and_dropout_semantics():
    x = torch.randn(6, 7, requires_grad=True)
    for mod, fn in [(nn.ReLU(), torch.relu), (nn.Sigmoid(), torch.sigmoid), (nn.Tanh(), torch.tanh),
                    (nn.GELU(), lambda t: torch.nn.functional.gelu(t, approximate="tanh")), (nn.SiLU(), torch.nn.functional.silu)]:
        y = mod(x)
        assert torch.allclose(y, fn(x), atol=1e-6)
        (g,) = torch.autograd.grad(y.sum(), x)
        (gr,) = torch.autograd.grad(fn(x).sum(), x)
        assert torch.allclose(g, gr, atol=1e-5)
    d = nn.Dropout(0.5)
    y = d(torch.ones(1000))
    assert 0.3 < float((y > 0).float().mean()) < 0.7 and torch.allclose(y[y > 0], torch.tensor(2.0))
    d.eval()
    assert torch.equal(d(torch.ones(10)), torch.ones(10))
    assert nn.Dropout(7.0).p == 1.0 and nn.Dropout(-1).p == 0.0
    fq = nn.FakeQuantize(8, 1.0)
    assert fq.qmin == -128 and fq.qmax == 127 and abs(fq.scale - 1 / 127) < 1e-9
    xq = torch.tensor([0.3, 5.0], requires_grad=True)
    fq(xq).sum().backward()
    assert xq.grad.tolist() == [1.0, 0.0]          # straight-through inside the clamp range only


def test_losses_match_reference_definitions():
    torch.manual_seed(1)
    p = torch.randn(8, 4, requires_grad=True); t = torch.randn(8, 4)
    assert torch.allclose(MSELoss()(p, t), ((p - t) ** 2).sum())                 # SUM, as in the reference
    assert torch.allclose(MSELoss("mean")(p, t), ((p - t) ** 2).mean())
    F = torch.nn.functional
    assert torch.allclose(L1Loss()(p, t), F.l1_loss(p, t))
    assert torch.allclose(HuberLoss(0.7)(p, t), F.huber_loss(p, t, delta=0.7), atol=1e-6)
    t01 = (t > 0).float()
    assert torch.allclose(BCEWithLogitsLoss()(p, t01), F.binary_cross_entropy_with_logits(p, t01), atol=1e-6)
    assert torch.allclose(BCELoss()(torch.sigmoid(p), t01), F.binary_cross_entropy(torch.sigmoid(p), t01), atol=1e-5)
    labels = torch.randint(0, 4, (8,))
    onehot = F.one_hot(labels, 4).float()
    assert torch.allclose(CrossEntropyLoss()(p, labels), F.cross_entropy(p, labels), atol=1e-6)
    assert torch.allclose(CrossEntropyLoss()(p, onehot), F.cross_entropy(p, labels), atol=1e-6)
    l = CrossEntropyLoss()(p, labels); l.backward()
    pr = p.detach().clone().requires_grad_(True); F.cross_entropy(pr, labels).backward()
    assert torch.allclose(p.grad, pr.grad, atol=1e-6)


def test_extreme_values_are_stable():
    big = torch.tensor([[1e4, -1e4, 0.0]], requires_grad=True)
    l = CrossEntropyLoss()(big, torch.tensor([0]))
    assert math.isfinite(float(l))
    assert torch.isfinite(nn.LayerNorm(3)(big)).all()
    assert torch.isfinite(nn.Sigmoid()(big)).all()


# ----------------------------------------------------------------------------- optimizers
def test_adam_reference_form_and_torch_form():
    torch.manual_seed(2)
    w0 = torch.randn(7, 3)
    grads = [torch.randn(7, 3) for _ in range(4)]
    p = torch.nn.Parameter(w0.clone()); opt = Adam([p], lr=1e-2)
    m = torch.zeros_like(w0); v = torch.zeros_like(w0); d = w0.clone()
    for t, g in enumerate(grads, 1):
        opt.zero_grad(); p.grad.copy_(g); opt.step()
        m = 0.9 * m + 0.1 * g; v = 0.999 * v + 0.001 * g * g
        lr_t = 1e-2 * math.sqrt(1 - 0.999 ** t) / (1 - 0.9 ** t)
        d = d - lr_t * m / (v.sqrt() + 1e-8)                       # rust-nn src/optim.rs:91-111
    assert torch.allclose(p.detach(), d, atol=1e-6)
    p2 = torch.nn.Parameter(w0.clone()); o2 = Adam([p2], lr=1e-2, torch_compat=True)
    pt = torch.nn.Parameter(w0.clone()); ot = torch.optim.Adam([pt], lr=1e-2)
    for g in grads:
        o2.zero_grad(); p2.grad.copy_(g); o2.step()
        pt.grad = g.clone(); ot.step()
    assert torch.allclose(p2.detach(), pt.detach(), atol=1e-6)


def test_sgd_rmsprop_muon_rules():
    w0 = torch.tensor([1.0, -2.0, 3.0]); g1 = torch.tensor([0.5, 0.5, -1.0]); g2 = torch.tensor([1.0, 0.0, 2.0])
    p = torch.nn.Parameter(w0.clone()); o = SGD([p], lr=0.1, momentum=0.9)
    o.zero_grad(); p.grad.copy_(g1); o.step()
    assert torch.allclose(p.detach(), w0 - 0.1 * g1)
    o.zero_grad(); p.grad.copy_(g2); o.step()
    assert torch.allclose(p.detach(), w0 - 0.1 * g1 - 0.1 * (0.9 * g1 + g2))
    p = torch.nn.Parameter(w0.clone()); o = RMSprop([p], lr=0.01)
    o.zero_grad(); p.grad.copy_(g1); o.step()
    v = 0.01 * g1 * g1
    assert torch.allclose(p.detach(), w0 - 0.01 * g1 / (v.sqrt() + 1e-8), atol=1e-6)
    p = torch.nn.Parameter(w0.clone()); o = Muon([p], lr=0.1, momentum=0.0)
    o.zero_grad(); p.grad.copy_(g1); o.step()
    rms = float((g1 * g1).mean().sqrt())
    assert torch.allclose(p.detach(), w0 - 0.1 * g1 / rms, atol=1e-6)
    W = torch.nn.Parameter(torch.randn(8, 4)); o = Muon([W], lr=0.1, mode="newton_schulz")
    o.zero_grad(); W.grad.copy_(torch.randn(8, 4)); before = W.detach().clone(); o.step()
    upd = (before - W.detach()) / 0.1
    s = torch.linalg.svdvals(upd)
    assert float(s.max()) < 2.0 and float(s.min()) > 0.3         # update is approximately orthogonal


def test_flat_params_fuse_groups_are_adjacent():
    mha = MultiHeadAttention(16, 2)
    opt = Adam(mha.parameters(), lr=1e-3)
    q, k, v = mha.q_proj.weight, mha.k_proj.weight, mha.v_proj.weight
    assert k.data_ptr() == q.data_ptr() + q.numel() * 4 and v.data_ptr() == k.data_ptr() + k.numel() * 4
    assert all(p.grad is not None and p._fused_grad for p in mha.parameters())
    x = torch.randn(2, 5, 16)
    mha(x).sum().backward()
    assert float(opt.flat.grad.abs().sum()) > 0


# ----------------------------------------------------------------------------- learning smoke tests
def test_xor_learns_on_cpu():
    torch.manual_seed(4)
    net = nn.Sequential(nn.Linear(2, 8), nn.Tanh(), nn.Linear(8, 1), nn.Sigmoid())
    x = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]]); y = torch.tensor([[0.], [1.], [1.], [0.]])
    tr = Trainer(net, Adam(net.parameters(), lr=0.05), MSELoss())
    loader = SimpleDataLoader(x, y, 4)
    loss = 1.0
    for _ in range(400):
        loss = tr.train_epoch(loader)
    assert loss < 0.1


def test_dataloader_batches():
    x = torch.arange(10.0).view(10, 1); y = torch.arange(10.0).view(10, 1)
    batches = list(SimpleDataLoader(x, y, 4))
    assert [b[0].shape[0] for b in batches] == [4, 4, 2]
    assert torch.equal(torch.cat([b[0] for b in batches]), x)          # no shuffle


def test_transformer_family_shapes_order_and_learning():
    torch.manual_seed(5)
    lt = LoopedTransformer(6, 16, 2, 32, 3, 2)
    x = torch.randn(2, 5, 6)
    out, loops = lt.forward_with_loops(x)
    assert out.shape == (2, 5, 3) and loops == 2
    n_block = len(TransformerBlock(16, 2, 32).parameters())
    assert n_block == 2 + 8 + 2 + 4
    assert len(lt.parameters()) == 2 + n_block + 2 + 2 + 4
    lt2 = LoopedTransformer(6, 16, 2, 32, 3, 4).with_adaptive_halting(0.5)
    out2, loops2 = lt2.forward_with_loops(x)
    assert 1 <= loops2 <= 4 and len(lt2.parameters()) == len(lt.parameters()) + 2
    tf = Transformer(6, 16, 2, 32, 3, 2).with_attention(AttentionKind.Flash)
    assert tf(x).shape == (2, 5, 3)
    opt = Adam(lt.parameters(), lr=1e-2)
    tgt = torch.randn(2, 5, 3)
    first = last = None
    for _ in range(30):
        opt.zero_grad(); l = MSELoss("mean")(lt(x), tgt); l.backward(); opt.step()
        first = first if first is not None else float(l); last = float(l)
    assert last < first


def test_mamba_family_shapes_order_and_learning():
    torch.manual_seed(6)
    blk = MambaBlock(8, 4, 2, 3)
    ps = blk.parameters()
    assert [tuple(p.shape) for p in ps] == [(16, 8), (16,), (16, 8), (16,), (16, 3), (16, 4), (16, 16), (16,), (4, 16), (4,), (4, 16), (4,), (8, 16), (8,)]
    assert torch.equal(blk.conv_weight[:, -1], torch.ones(16)) and float(blk.conv_weight[:, :-1].abs().sum()) == 0
    assert torch.allclose(blk.a[0], torch.tensor([-0.5, -1.0, -1.5, -2.0]))
    m = Mamba(8, 4, 2, 3, 2)
    x = torch.randn(2, 6, 8)
    assert m(x).shape == (2, 6, 8)
    h = HybridMamba(8).with_mamba(4, 2, 3).with_layer(nn.Sequential(nn.Linear(8, 8), nn.ReLU()))
    assert h(x).shape == (2, 6, 8)
    lm = MambaLM(50, 16, 2, d_state=4, d_conv=3, expand=2, dt_rank=2)
    ids = torch.randint(0, 50, (2, 12)); lab = torch.randint(0, 50, (2, 12))
    opt = Adam(lm.parameters(), lr=5e-3)
    losses = []
    for _ in range(25):
        opt.zero_grad(); l = lm.loss(ids, lab); l.backward(); opt.step(); losses.append(float(l))
    assert losses[-1] < losses[0]


# ----------------------------------------------------------------------------- checkpoints
def test_rnnb_golden_bytes_and_roundtrip():
    t = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    buf = serialize.serialize([("w", t)])
    golden = (b"RNNB" + struct.pack("<II", 1, 1) + struct.pack("<I", 1) + b"w" + struct.pack("<I", 2) + struct.pack("<QQ", 2, 3)
              + struct.pack("<I", 6) + struct.pack("<6f", 1, 2, 3, 4, 5, 6))
    assert buf == golden
    (name, back), = serialize.deserialize(buf)
    assert name == "w" and back.requires_grad and torch.equal(back.detach(), t)
    with pytest.raises(SerializationError):
        serialize.deserialize(b"XXXX" + buf[4:])
    with pytest.raises(SerializationError):
        serialize.deserialize(buf[:-3])
    with pytest.raises(SerializationError):
        serialize.deserialize(b"RNNB" + struct.pack("<II", 2, 0))
    scalar = serialize.deserialize(serialize.serialize([("s", torch.tensor(3.5))]))[0][1]
    assert scalar.shape == () and float(scalar) == 3.5


def test_save_load_model_and_resume(tmp_path):
    torch.manual_seed(7)
    make = lambda: nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))
    a, b = make(), make()
    blob = serialize.save_model(a)
    names = [n for n, _ in serialize.deserialize(blob)]
    assert names == ["param_0", "param_1", "param_2", "param_3"]
    serialize.load_model(b, blob)
    assert all(torch.equal(p, q) for p, q in zip(a.parameters(), b.parameters()))
    with pytest.raises(SerializationError):
        serialize.load_model(nn.Sequential(nn.Linear(4, 8)), blob)
    # train N, save, reload, train M  ==  train N + M
    x = torch.randn(16, 4); y = torch.randint(0, 2, (16,))
    def steps(model, opt, n):
        for _ in range(n):
            opt.zero_grad(); CrossEntropyLoss()(model(x), y).backward(); opt.step()
    m1 = make(); serialize.load_model(m1, blob); o1 = Adam(m1.parameters(), lr=1e-2); steps(m1, o1, 7)
    m2 = make(); serialize.load_model(m2, blob); o2 = Adam(m2.parameters(), lr=1e-2); steps(m2, o2, 3)
    path = str(tmp_path / "ck.rnnb")
    serialize.save_checkpoint(path, m2, o2)
    m3 = make(); o3 = Adam(m3.parameters(), lr=1e-2)
    serialize.load_checkpoint(path, m3, o3)
    steps(m3, o3, 4)
    assert all(torch.allclose(p, q, atol=1e-6) for p, q in zip(m1.parameters(), m3.parameters()))


def test_safetensors_roundtrip_skips_metadata():
    named = [("a.weight", torch.randn(3, 4)), ("b", torch.randn(5))]
    blob = serialize.safetensors_export(named)
    back = serialize.safetensors_import(blob)
    assert [n for n, _ in back] == ["a.weight", "b"]
    assert all(torch.equal(x[1], y[1]) for x, y in zip(named, back))
    import json
    hdr = json.dumps({"__metadata__": {"format": "pt"}, "z": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    blob2 = struct.pack("<Q", len(hdr)) + hdr + struct.pack("<2f", 1.5, -2.0)
    (n, t), = serialize.safetensors_import(blob2)
    assert n == "z" and t.tolist() == [1.5, -2.0]


# ----------------------------------------------------------------------------- positional encodings
def test_rope_properties_and_gradient():
    r = RoPE.new(8, 16)
    x = torch.randn(2, 3, 10, 8, requires_grad=True)
    y = r.apply(x)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)      # rotation preserves norms
    assert torch.allclose(y[:, :, 0], x[:, :, 0], atol=1e-6)              # position 0 is the identity
    w = torch.randn_like(y)
    (g,) = torch.autograd.grad((y * w).sum(), x)
    eps = 1e-3
    xp = x.detach().clone(); xp[0, 0, 3, 2] += eps
    xm = x.detach().clone(); xm[0, 0, 3, 2] -= eps
    num = float(((r.apply(xp) - r.apply(xm)) * w).sum()) / (2 * eps)
    assert abs(num - float(g[0, 0, 3, 2])) < 1e-2
    with pytest.raises(ValueError):
        r.apply(torch.randn(1, 17, 8))
    r.extend(32)
    assert r.apply(torch.randn(1, 20, 8)).shape == (1, 20, 8)
    yarn = RoPE.yarn(8, 16, 10000.0, 4.0)
    assert float(yarn.inv_freq[-1]) < float(r.inv_freq[-1])               # lower frequencies with a scaled base


def test_alibi_sinusoidal_learned_carope():
    a = AlibiBias(4)
    assert abs(a.slope(0) - 2 ** (-2.0)) < 1e-7 and a.slope(9) == 0.0
    m = a.bias_matrix(5)
    assert m.shape == (4, 5, 5) and float(m[0, 0, 3]) == -a.slope(0) * 3 and float(m.max()) == 0.0
    s = SinusoidalPE(6, 10)
    assert s.table().shape == (10, 6) and float(s.table()[0, 1]) == 1.0 and float(s.table()[0, 0]) == 0.0
    x = torch.zeros(2, 4, 6)
    assert torch.allclose(s.apply(x)[0], s.table()[:4])
    l = LearnedPE(6, 10).init_sinusoidal()
    assert torch.allclose(l.apply(x)[1], s.table()[:4]) and len(l.parameters()) == 1
    c = CARoPE(8, 5, 12).with_spread(0.2)
    out = c.apply(torch.randn(2, 7, 8), torch.randn(7, 5))
    assert out.shape == (2, 7, 8) and len(c.parameters()) == 1


def test_dact_colsum_and_add_layernorm_reference_paths():
    """CPU restatements of the two streaming kernels that took work out of GEMM epilogues."""
    import torch
    from rust_neural_network_b200.ops import gemm as G
    from rust_neural_network_b200.ops import kernels as K
    torch.manual_seed(0)
    g, pre = torch.randn(37, 24), torch.randn(37, 24)
    for act in ("relu", "gelu", "silu"):
        want = g * G.dact_ref(pre, act)
        acc = torch.ones(24)
        got, none = K.dact_colsum(g.clone(), pre, act, bias_grad=acc)
        assert none is None and torch.allclose(got, want, atol=1e-5)
        assert torch.allclose(acc, 1.0 + want.sum(0), atol=1e-4)
        got2, db = K.dact_colsum(g.clone(), pre, act)
        assert torch.allclose(db, want.sum(0), atol=1e-4) and torch.allclose(got2, want, atol=1e-5)
    x, r = torch.randn(9, 16), torch.randn(9, 16)
    gamma, beta = torch.rand(16) + 0.5, torch.randn(16)
    s, y, mean, rstd = K.add_layernorm_fwd(x, r, gamma, beta, 1e-5)
    assert torch.allclose(s, x + r) and torch.allclose(y, torch.nn.functional.layer_norm(x + r, (16,), gamma, beta, 1e-5), atol=1e-5)
    assert torch.allclose(mean, (x + r).mean(1), atol=1e-6)
