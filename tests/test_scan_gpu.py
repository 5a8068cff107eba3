"""Selective scan / causal conv1d kernels against the sequential fp32 PyTorch reference
(forward values and every gradient), including odd sizes (rust-nn tests/selective_scan.rs uses
finite differences on tiny shapes; here the oracle is autograd through the fp32 recurrence)."""
import pytest
import torch

from rust_neural_network_b200.ops import scan as SC

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-9))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,S,D,N,full", [(2, 64, 128, 16, True), (1, 37, 70, 8, True), (2, 130, 256, 16, False), (1, 8, 33, 4, True),
                                          (1, 45, 70, 16, True), (3, 257, 100, 16, True), (2, 1024, 64, 16, False)])
def test_selective_scan_fwd_bwd(B, S, D, N, full, dtype):
    torch.manual_seed(0)
    dev = "cuda"
    u = torch.randn(B, S, D, device=dev); delta = torch.randn(B, S, D, device=dev) * 0.5
    A = -(torch.rand(D, N, device=dev) * 2 + 0.2)
    Bm = torch.randn(B, S, N, device=dev); Cm = torch.randn(B, S, N, device=dev)
    Dskip = torch.randn(D, device=dev) if full else None
    z = torch.randn(B, S, D, device=dev) if full else None
    dbias = torch.randn(D, device=dev) * 0.3 if full else None
    softplus = full
    if not full:
        delta = delta.abs() + 0.05
    cast = lambda t: t.to(dtype) if t is not None else None
    ins_k = [cast(u), cast(delta), A.clone(), cast(Bm), cast(Cm), Dskip.clone() if full else None, cast(z), dbias.clone() if full else None]
    ins_r = [t.float().clone() if t is not None else None for t in ins_k]
    for t in ins_k + ins_r:
        if t is not None:
            t.requires_grad_(True)
    y = SC.selective_scan(*ins_k, softplus)
    yr = SC.selective_scan_ref(*ins_r, softplus)
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-4
    assert rel_err(y, yr) < tol
    w = torch.randn_like(yr)
    (y.float() * w).sum().backward()
    (yr * w).sum().backward()
    names = ["u", "delta", "A", "B", "C", "D", "z", "dbias"]
    gtol = 6e-2 if dtype == torch.bfloat16 else 2e-3
    for nm, a, b in zip(names, ins_k, ins_r):
        if a is None:
            continue
        assert a.grad is not None, nm
        assert rel_err(a.grad, b.grad) < gtol, nm


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,S,C,K,act,bias", [(2, 100, 192, 4, "silu", True), (1, 33, 70, 3, "none", False), (2, 64, 128, 2, "silu", False), (1, 200, 64, 4, "none", True)])
def test_causal_conv1d(B, S, C, K, act, bias, dtype):
    torch.manual_seed(1)
    dev = "cuda"
    x = torch.randn(B, S, C, device=dev).to(dtype).requires_grad_(True)
    w = (torch.randn(C, K, device=dev) * 0.5).requires_grad_(True)
    b = (torch.randn(C, device=dev) * 0.2).requires_grad_(True) if bias else None
    y = SC.causal_conv1d(x, w, b, act)
    xr = x.detach().float().requires_grad_(True); wr = w.detach().clone().requires_grad_(True)
    br = b.detach().clone().requires_grad_(True) if bias else None
    yr = SC.causal_conv1d_ref(xr, wr, br, act)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert rel_err(y, yr) < tol
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward(); (yr * g).sum().backward()
    gtol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert rel_err(x.grad, xr.grad) < gtol
    assert rel_err(w.grad, wr.grad) < gtol
    if bias:
        assert rel_err(b.grad, br.grad) < gtol


@pytest.mark.gpu
def test_selective_scan_recompute_gives_identical_gradients():
    """`recompute=True` keeps no state checkpoints and rebuilds them in the backward: same bits, less memory held."""
    from rust_neural_network_b200.ops.scan import selective_scan
    torch.manual_seed(0)
    B, S, D, N = 2, 300, 128, 16
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.5).bfloat16()
    u, dl, z, Bm, Cm = mk(B, S, D), mk(B, S, D), mk(B, S, D), mk(B, S, N), mk(B, S, N)
    A = -torch.arange(1, N + 1, device="cuda", dtype=torch.float32).repeat(D, 1)
    Dk, db = torch.randn(D, device="cuda"), torch.randn(D, device="cuda") * 0.1
    res = []
    for rec in (False, True):
        ins = [t.clone().requires_grad_(True) for t in (u, dl, A, Bm, Cm, Dk, z, db)]
        y = selective_scan(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], ins[6], ins[7], True, rec)
        y.float().square().sum().backward()
        res.append([y.detach()] + [t.grad for t in ins])
    for a, b in zip(*res):
        assert torch.equal(a, b)
