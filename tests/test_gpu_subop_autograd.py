"""Gradients through the three fused sub-ops that the reference wraps in autograd Functions
(FusedSwiGLUFFNFwd lact_swiglu_ffn.py:19-76, FusedLactSwiGLUFFNBwd lact_fw_grad.py:21-156,
L2NormAddFunction l2norm_triton_kernels.py:386-416), against autograd through the fp32
restatement of the same formulas on the same bf16-rounded inputs.  The backward kernels recompute
pre-activations in bf16 as the reference's do: bf16 tolerance (max|a-ref|/max|ref| <= 2e-2,
cosine >= 0.999; fp32 row sums for the learning rates)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def lb():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    import lact_b200
    return lact_b200


@pytest.fixture(scope="module")
def orc():
    from oracle import lact_oracle
    return lact_oracle


def _check(orc, got, ref, what, tol=2e-2, cos=0.999):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    rm, cs = orc.rel_max(got, ref), orc.cosine(got, ref)
    assert rm <= tol and cs >= cos, f"{what}: rel_max={rm:.3e} cos={cs:.6f}"


def _mk(B, N, D, H, seed):
    g = torch.Generator().manual_seed(seed)
    w02 = (torch.randn(B, 2 * H, D, generator=g) / D ** 0.5).to(BF16)
    w1 = (torch.randn(B, D, H, generator=g) / H ** 0.5).to(BF16)
    x = torch.randn(B, N, D, generator=g).to(BF16)
    v = torch.randn(B, N, D, generator=g).to(BF16)
    lr = [torch.nn.functional.softplus(torch.randn(B, N, generator=g) - 2.0) for _ in range(3)]
    return w02, w1, x, v, lr, g


@pytest.mark.parametrize("B,N,D,H", [(2, 300, 64, 128), (1, 512, 384, 384)])
def test_fused_swiglu_ffn_fwd_is_differentiable(lb, orc, B, N, D, H):
    w02, w1, x, _, _, g = _mk(B, N, D, H, seed=41)
    dO = torch.randn(B, N, D, generator=g).to(BF16)
    # fp32 autograd through the formula of reference_swiglu_ffn_fwd (lact_swiglu_ffn.py:104-116)
    a, b, c = (t.float().clone().requires_grad_(True) for t in (w02, w1, x))
    y0, y2 = c @ a[:, :H].transpose(1, 2), c @ a[:, H:].transpose(1, 2)
    o_ref = (torch.nn.functional.silu(y0) * y2) @ b.transpose(1, 2)
    (o_ref * dO.float()).sum().backward()
    ca, cb, cc = (t.cuda().clone().requires_grad_(True) for t in (w02, w1, x))
    o = lb.fused_swiglu_ffn_fwd(ca, cb, cc)
    _check(orc, o, o_ref, "o")
    o.backward(dO.cuda())
    lb.synchronize_and_check()
    for got, ref, name in ((ca.grad, a.grad, "grad W0_W2"), (cb.grad, b.grad, "grad W1"), (cc.grad, c.grad, "grad X")):
        assert got.dtype == BF16
        _check(orc, got, ref, name)


@pytest.mark.parametrize("B,N,D,H", [(2, 300, 64, 128), (1, 512, 384, 384)])
def test_fast_weight_grads_are_differentiable(lb, orc, B, N, D, H):
    w02, w1, k, v, lr, g = _mk(B, N, D, H, seed=42)
    g02 = torch.randn(B, 2 * H, D, generator=g).to(BF16)
    g1 = torch.randn(B, D, H, generator=g).to(BF16)
    leaves = [t.float().clone().requires_grad_(True) for t in (w02, w1, k, v, *lr)]
    dw02_ref, dw1_ref = orc.grads_fused(*leaves)  # fp32 inputs: the formula without roundings
    ((dw02_ref * g02.float()).sum() + (dw1_ref * g1.float()).sum()).backward()
    cl = [t.cuda().clone().requires_grad_(True) for t in (w02, w1, k, v, *lr)]
    dw02, dw1 = lb.fused_lact_swiglu_ffn_fast_weight_grads(*cl)
    _check(orc, dw02, dw02_ref, "DW0_DW2")
    _check(orc, dw1, dw1_ref, "DW1")
    torch.autograd.backward([dw02, dw1], [g02.cuda(), g1.cuda()])
    lb.synchronize_and_check()
    for got, ref, name in zip(cl, leaves, ("W0_W2", "W1", "K", "V", "lr0", "lr1", "lr2")):
        assert got.grad is not None, name
        assert got.grad.shape == got.shape
        _check(orc, got.grad, ref.grad, "grad " + name, tol=3e-2 if name.startswith("lr") else 2e-2)
    # one output unused: its cotangent is absent, not a materialised zero tensor
    cl2 = [t.cuda().clone().requires_grad_(True) for t in (w02, w1, k, v, *lr)]
    only02, _ = lb.fused_lact_swiglu_ffn_fast_weight_grads(*cl2)
    only02.backward(g02.cuda())
    assert torch.isfinite(cl2[2].grad.float()).all()


@pytest.mark.parametrize("x_dtype,add_dtype,tgt", [(torch.float32, BF16, None), (torch.float32, BF16, BF16),
                                                  (BF16, BF16, None),
                                                  # both fp32: the two gradients are the same values, yet two tensors
                                                  (torch.float32, torch.float32, None)])
def test_l2_norm_add_fused_is_differentiable(lb, orc, x_dtype, add_dtype, tgt):
    B, T, D = 3, 200, 384
    g = torch.Generator().manual_seed(43)
    x = (torch.randn(B, T, D, generator=g) / D ** 0.5).to(x_dtype)
    xa = (torch.randn(B, T, D, generator=g) * 0.05).to(add_dtype)
    sc = torch.rand(B, T, generator=g) + 0.5
    dy = torch.randn(B, T, D, generator=g)
    a, b, c = (t.float().clone().requires_grad_(True) for t in (x, xa, sc))
    y_ref = orc.l2_norm_add(a, b, c)
    (y_ref * dy).sum().backward()
    ca, cb, cc = (t.cuda().clone().requires_grad_(True) for t in (x, xa, sc))
    y = lb.l2_norm_add_fused(ca, cb, cc, tgt_dtype=tgt)
    assert y.dtype == (tgt if tgt is not None else x_dtype)
    _check(orc, y, y_ref, "y", tol=1e-2 if y.dtype == BF16 else 1e-5)
    y.backward(dy.cuda().to(y.dtype))
    lb.synchronize_and_check()
    tol = 1e-2 if BF16 in (x_dtype, tgt) else 2e-5
    assert ca.grad.dtype == x_dtype and cb.grad.dtype == add_dtype
    _check(orc, ca.grad, a.grad, "dx", tol=tol)
    _check(orc, cb.grad, b.grad, "dx_add", tol=1e-2)
    _check(orc, cc.grad, c.grad, "dtgt_scale", tol=tol)
