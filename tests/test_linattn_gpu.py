"""Fused causal linear attention (csrc/attention/linattn_sm100.cu) against the fp32 O(S^2) oracle: forward and all three
gradients, both feature maps, head sizes 64 and 128, sequence lengths that are not chunk multiples, a long sequence where
the state carries most of the mass, the state-in / state-out interface a sequence-parallel rank uses, and bit-exact
repeatability (nothing in these kernels accumulates with atomics)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def _inputs(B, S, H, d, seed=0):
    g = torch.Generator().manual_seed(seed)
    mk = lambda: (torch.randn(B, S, H, d, generator=g) * 0.7).to(torch.bfloat16).cuda()
    return mk(), mk(), mk(), mk()


def _grads(fn, q, k, v, w, as_float):
    ins = [(t.float() if as_float else t).clone().requires_grad_(True) for t in (q, k, v)]
    out = fn(*ins)
    out.backward(w.float() if as_float else w)
    return out.detach(), [t.grad for t in ins]


def _check(S, hd, kind, B=2, H=3, seed=0):
    """Two oracles. (1) fp32 everything. (2) fp32 arithmetic on bf16-ROUNDED feature maps: the function a kernel with bf16
    tensor-core operands evaluates. dQ and dK are differences of nearly equal sums over the features; ELU + 1 features sit
    near 1, where bf16 resolves 2^-8, so the rounding of the operands alone moves dQ by a few per cent against (1). Against
    (2) only the kernel's own arithmetic is left (fp32 state; state, masked tile and O carried as value + remainder)."""
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops.linear_attention import FusedCausalLinearAttnFn, linear_attention_ref
    q, k, v, w = _inputs(B, S, H, hd, seed)
    scale = hd ** -0.5
    out, g = _grads(lambda a, b, c: FusedCausalLinearAttnFn.apply(a, b, c, scale, 1e-6, kind, None), q, k, v, w, False)
    torch.cuda.synchronize(); nv.check_status()
    ref, gr = _grads(lambda a, b, c: linear_attention_ref(a, b, c, scale=scale, causal=True, kind=kind), q, k, v, w, True)
    rnd, gb = _grads(lambda a, b, c: linear_attention_ref(a, b, c, scale=scale, causal=True, kind=kind, feature_dtype=torch.bfloat16), q, k, v, w, True)
    e32 = {n: _rel(a, b) for n, a, b in zip(("dq", "dk", "dv"), g, gr)}
    e16 = {n: _rel(a, b) for n, a, b in zip(("dq", "dk", "dv"), g, gb)}
    assert _rel(out, ref) < 1e-2
    return e32, e16


@pytest.mark.parametrize("S,hd", [(128, 64), (300, 64), (1024, 64), (257, 128), (1024, 128)])
@pytest.mark.parametrize("kind", ["elu", "relu2"])
def test_fused_forward_backward_match_fp32_oracle(S, hd, kind):
    e32, e16 = _check(S, hd, kind)
    # the kernel's own arithmetic (fp32 state, value + remainder operands): 0.25 % measured on every case
    assert all(e < 6e-3 for e in e16.values()), ("vs fp32 arithmetic on bf16 features", e16)
    assert e32["dk"] < 8e-3 and e32["dv"] < 8e-3, e32
    # rounding phi(Q), phi(K) to bf16 is what is left against the all-fp32 oracle: 2-3 % of dQ for ELU + 1 (features near 1)
    assert e32["dq"] < (8e-3 if kind == "relu2" else 4.5e-2), e32


def test_long_sequence_gradients():
    """8192 tokens: almost all of every output comes through the carried state (64 chunks)."""
    e32, e16 = _check(8192, 64, "elu", B=1, H=2, seed=3)
    assert all(e < 6e-3 for e in e16.values()), e16
    assert e32["dk"] < 8e-3 and e32["dv"] < 8e-3 and e32["dq"] < 4e-2, e32
    e32, e16 = _check(8192, 64, "relu2", B=1, H=2, seed=3)
    assert all(e < 8e-3 for e in e32.values()), e32


def test_state_in_state_out_equals_one_long_sequence():
    """Two slices chained through s_out -> s_in (forward) and ds_out -> ds_in (backward) reproduce the unsplit run: what
    a sequence-parallel rank does with the exchanged states."""
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops import linear_attention as LA
    B, S, H, d = 2, 768, 2, 64
    q, k, v, w = _inputs(B, S, H, d, seed=5)
    full_in = [t.clone().requires_grad_(True) for t in (q, k, v)]
    full = LA.FusedCausalLinearAttnFn.apply(*full_in, 0.125, 1e-6, "elu", None)
    full.backward(w)
    h = 384
    lo, hi = slice(0, h), slice(h, S)
    st = torch.empty(B * H, d * d + d, device="cuda")
    o0, o1 = torch.empty_like(q[:, lo]), torch.empty_like(q[:, hi])
    den0, den1 = torch.empty(B, H, h, device="cuda"), torch.empty(B, H, S - h, device="cuda")
    cq, ck, cv, cw = (lambda s: [t[:, s].contiguous() for t in (q, k, v, w)])(lo)
    dq_, dk_, dv_, dw_ = (lambda s: [t[:, s].contiguous() for t in (q, k, v, w)])(hi)
    LA._launch(0, cq, ck, cv, 0.125, 1e-6, "elu", o=o0, den=den0, s_out=st)
    LA._launch(0, dq_, dk_, dv_, 0.125, 1e-6, "elu", o=o1, den=den1, s_in=st)
    assert _rel(torch.cat([o0, o1], 1), full) < 2e-3
    # backward: the later slice first, its dS / dz flow into the earlier one
    g = {n: torch.empty_like(q) for n in ("dq", "dk", "dv")}
    dst = torch.empty_like(st)
    gq1, gk1, gv1 = (torch.empty_like(o1) for _ in range(3))
    LA._launch(1, dq_, dk_, dv_, 0.125, 1e-6, "elu", o=o1, den=den1, dout=dw_, dq=gq1, s_in=st)
    LA._launch(2, dq_, dk_, dv_, 0.125, 1e-6, "elu", o=o1, den=den1, dout=dw_, dk=gk1, dv=gv1, ds_out=dst)
    gq0, gk0, gv0 = (torch.empty_like(o0) for _ in range(3))
    LA._launch(1, cq, ck, cv, 0.125, 1e-6, "elu", o=o0, den=den0, dout=cw, dq=gq0)
    LA._launch(2, cq, ck, cv, 0.125, 1e-6, "elu", o=o0, den=den0, dout=cw, dk=gk0, dv=gv0, ds_in=dst)
    torch.cuda.synchronize(); nv.check_status()
    for a, b, name in ((torch.cat([gq0, gq1], 1), full_in[0].grad, "dq"), (torch.cat([gk0, gk1], 1), full_in[1].grad, "dk"),
                       (torch.cat([gv0, gv1], 1), full_in[2].grad, "dv")):
        assert _rel(a, b) < 4e-2, (name, _rel(a, b))        # the chained launches run without the remainder of O
    # the state-only pass yields the same total state as the full pass
    st2 = torch.empty_like(st)
    LA._launch(0, cq, ck, cv, 0.125, 1e-6, "elu", s_out=st2, state_only=True)
    torch.cuda.synchronize()
    assert _rel(st2, st) < 1e-5


def test_run_twice_is_bit_identical():
    from rust_neural_network_b200.ops.linear_attention import FusedCausalLinearAttnFn
    q, k, v, w = _inputs(2, 640, 2, 64, seed=9)
    res = []
    for _ in range(2):
        qi, ki, vi = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = FusedCausalLinearAttnFn.apply(qi, ki, vi, 0.125, 1e-6, "elu", None)
        out.backward(w)
        res.append((out.detach().clone(), qi.grad.clone(), ki.grad.clone(), vi.grad.clone()))
    for a, b in zip(*res):
        assert torch.equal(a, b)
