"""Training backward (Muon off) against autograd through the CPU oracle.

The oracle runs the reference's unfused arithmetic in fp32 on the same bf16-rounded inputs;
the CUDA backward recomputes pre-activations in bf16 (as the reference's fused backward does),
so gradients agree to bf16 accuracy: max|a-ref|/max|ref| <= 3e-2 and cosine >= 0.999.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
NAMES = ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")


@pytest.fixture(scope="module")
def lb():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    import lact_b200
    return lact_b200


def _grads_oracle(orc, inp, fn, mom, dO):
    leaves = {n: inp[n].float().clone().requires_grad_(True) for n in NAMES}
    m = inp["momentum"].clone().requires_grad_(True) if mom else None
    o = fn(*[leaves[n] for n in NAMES], m)
    (o * dO.float()).sum().backward()
    g = {n: leaves[n].grad for n in NAMES}
    if mom:
        g["momentum"] = m.grad
    return o.detach(), g


def _grads_cuda(inp, fn, mom, dO):
    leaves = {n: inp[n].cuda().clone().requires_grad_(True) for n in NAMES}
    m = inp["momentum"].cuda().clone().requires_grad_(True) if mom else None
    o = fn(*[leaves[n] for n in NAMES], m)
    (o.float() * dO.cuda().float()).sum().backward()
    g = {n: leaves[n].grad for n in NAMES}
    if mom:
        g["momentum"] = m.grad
    return o.detach(), g


def _check(orc, got, ref, names, tol=3e-2, cos=0.999):
    for n in names:
        a, b = got[n].float().cpu(), ref[n].float()
        assert a.shape == b.shape, n
        assert torch.isfinite(a).all(), n
        rm, cs = orc.rel_max(a, b), orc.cosine(a, b)
        # the momentum gradient is one scalar per (entry, chunk), a long bf16-operand reduction: wider band
        t = 8e-2 if n == "momentum" else tol
        assert rm <= t and cs >= cos, f"grad {n}: rel_max={rm:.3e} cos={cs:.6f}"


@pytest.mark.parametrize("mom", [False, True])
@pytest.mark.parametrize("shape", [(2, 576, 64, 64, 128), (1, 700, 128, 64, 256)])
def test_llm_postnorm_backward_muon_off(lb, mom, shape):
    from oracle import lact_oracle as orc
    B, L, D, H, C = shape
    inp = orc.make_inputs(B, L, D, H, seed=21)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(3)).to(BF16)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.block_causal_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=False, momentum=m)
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.block_causal_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=False, momentum=m)
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, mom, dO)
    o, g = _grads_cuda(inp, cu_fn, mom, dO)
    assert orc.rel_max(o.float().cpu(), o_ref) <= 2e-2
    _check(orc, g, g_ref, list(NAMES) + (["momentum"] if mom else []))
    assert g["q"].dtype == BF16 and g["w0"].dtype == torch.float32 and g["lr0"].shape == inp["lr0"].shape


def test_fused_signature_backward_muon_off(lb):
    """eps-inside renorm (fused post-norm signature): gradients vs autograd through the oracle's
    restatement of the fused path."""
    from oracle import lact_oracle as orc
    B, L, D, H, C = 2, 512, 64, 128, 128
    inp = orc.make_inputs(B, L, D, H, seed=22)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(4)).to(BF16)

    def ref_fn(w0, w1, w2, q, k, v, l0, l1, l2, m):
        # fp32 arithmetic with the fused path's semantics (eps inside the square root)
        cfg = orc.ScanConfig(use_muon=False, renorm="inner", fp32_mode=True)
        steps = [("apply", s, s + C, s) if kind == 0 else ("update", s, s + C, 0)
                 for kind, s in [(0, 0), (1, 0), (0, 128), (1, 128), (0, 256), (1, 256), (0, 384)]]
        o, *_ = scan_autograd(orc, w0, w1, w2, q, k, v, l0, l1, l2, steps, cfg, m)
        return o

    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=False, momentum=m)
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, True, dO)
    o, g = _grads_cuda(inp, cu_fn, True, dO)
    _check(orc, g, g_ref, list(NAMES) + ["momentum"])


def scan_autograd(orc, w0, w1, w2, q, k, v, l0, l1, l2, steps, cfg, m):
    """Differentiable fp32 version of the oracle's scan model (no in-place writes)."""
    import torch.nn.functional as F
    n0, n1, n2 = (w.norm(dim=2, keepdim=True) for w in (w0, w1, w2))
    outs = []
    ms = None
    if m is not None:
        ms = [torch.zeros_like(w0), torch.zeros_like(w1), torch.zeros_like(w2)]
    nm = orc.Numerics("ref")
    for kind, s, e, _ in steps:
        if kind == "apply":
            outs.append(orc.apply_ref(w0, w1, w2, q[:, s:e], nm))
            continue
        d0, d1, d2 = orc.grads_ref(w0, w1, w2, k[:, s:e], v[:, s:e], l0[:, s:e], l1[:, s:e], l2[:, s:e], nm)
        if ms is not None:
            beta = m[:, s:e].mean(dim=1, keepdim=True)
            d0, d1, d2 = d0 + ms[0] * beta, d1 + ms[1] * beta, d2 + ms[2] * beta
            ms = [d0, d1, d2]
        norm = lambda w, n: w * (1 / torch.sqrt(torch.sum(w * w, dim=2, keepdim=True) + 1e-5)) * n
        w0, w1, w2 = norm(w0 + d0, n0), norm(w1 + d1, n1), norm(w2 + d2, n2)
    return torch.cat(outs, dim=1), w0, w1, w2


@pytest.mark.parametrize("mom", [False, True])
def test_llm_prenorm_backward_muon_off(lb, mom):
    """Pre-norm recurrence (un-normalised master copy, ttt_operation.py:217-364)."""
    from oracle import lact_oracle as orc
    B, L, D, H, C = 2, 576, 64, 64, 128
    inp = orc.make_inputs(B, L, D, H, seed=24)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(6)).to(BF16)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.block_causal_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=False, momentum=m, prenorm=True)
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.prenorm_block_causal_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=False, momentum=m)
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, mom, dO)
    o, g = _grads_cuda(inp, cu_fn, mom, dO)
    assert orc.rel_max(o.float().cpu(), o_ref) <= 2e-2
    _check(orc, g, g_ref, list(NAMES) + (["momentum"] if mom else []))


def test_prenorm_fused_signature_backward_runs_with_muon(lb):
    """bf16 normalised copy + Muon + momentum: finite gradients of the right shapes, and the
    same gradients as the unfused pre-norm signature up to the bf16 copy."""
    from oracle import lact_oracle as orc
    B, L, D, H, C = 1, 384, 64, 64, 128
    inp = orc.make_inputs(B, L, D, H, seed=25)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(7)).to(BF16)
    fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.prenorm_block_causal_lact_swiglu_fused_kernel_triton(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=True, momentum=m)
    o, g = _grads_cuda(inp, fn, True, dO)
    for n in list(NAMES) + ["momentum"]:
        assert g[n] is not None and torch.isfinite(g[n]).all(), n
    assert g["q"].shape == inp["q"].shape and g["w1"].shape == inp["w1"].shape
    # tokens of chunk 0 see the initial weights only: their dq equals the Muon-off dq
    fn0 = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.prenorm_block_causal_lact_swiglu_fused_kernel_triton(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=False, momentum=m)
    _, g0 = _grads_cuda(inp, fn0, True, dO)
    assert torch.equal(g["q"][:, :C], g0["q"][:, :C])
    # and against autograd through the oracle's pre-norm fused recurrence run with the kernels' rounding model of the
    # iteration (three chunks, two updates: the un-normalised masters are rebuilt from the kept results)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.block_causal_lact_swiglu_fused(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=True, momentum=m, prenorm=True,
        ns=orc.newton_schulz_folded)
    _, g_ref = _grads_oracle(orc, inp, ref_fn, True, dO)
    for n in NAMES:
        a, b = g[n].float().cpu(), g_ref[n].float()
        assert orc.cosine(a, b) >= 0.99, (n, orc.cosine(a, b))
        assert orc.rel_fro(a, b) <= 0.15, (n, orc.rel_fro(a, b))


@pytest.mark.parametrize("muon", [False, True])
def test_bidirectional_backward(lb, muon):
    """minimal_implementations/bidirectional_lact_layer.py:73-160 with gradients.  With Muon the
    weights are overwritten, w <- renorm(NS(dw) + dw): the gradient reaches the initial weights
    only through dw (and the target norms)."""
    from oracle import lact_oracle as orc
    B, L, D, H = 2, 256, 64, 64
    inp = orc.make_inputs(B, L, D, H, seed=26)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(8)).to(BF16)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.bidirectional_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, use_muon=muon)
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.bidirectional_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, use_muon=muon)
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, False, dO)
    o, g = _grads_cuda(inp, cu_fn, False, dO)
    if not muon:
        _check(orc, g, g_ref, list(NAMES))
        return
    for n in NAMES:  # one bf16 Newton-Schulz pass (5 iterations) between inputs and output; measured: cosine
        a, b = g[n].float().cpu(), g_ref[n].float()   # >= 0.9984, rel_fro <= 0.057 against the eager-rounding oracle
        assert torch.isfinite(a).all(), n
        assert orc.cosine(a, b) >= 0.995, (n, orc.cosine(a, b))
        assert orc.rel_fro(a, b) <= 0.12, (n, orc.rel_fro(a, b))


@pytest.mark.parametrize("shape,steps", [((3, 64, 64), None), ((2, 64, 128), 5), ((2, 128, 64), 3), ((2, 192, 192), None)])
def test_newton_schulz_backward(lb, shape, steps):
    """d NS(G) / dG applied to a random cotangent: against autograd through an fp64 iteration.
    The reference differentiates its bf16 iteration, whose own gradient deviates from the fp64
    one by the amount measured here; the kernel path must not be worse than 1.5x that."""
    from oracle import lact_oracle as orc
    from lact_b200 import backward as bw
    g = torch.Generator().manual_seed(7)
    G = torch.randn(*shape, generator=g)
    dU = torch.randn(*shape, generator=g)

    def autograd_of(fn, dtype):
        Gl = G.to(BF16).to(dtype).clone().requires_grad_(True)
        (fn(Gl, steps).to(dtype) * dU.to(dtype)).sum().backward()
        return Gl.grad.double()

    ref64 = autograd_of(orc.newton_schulz_f64, torch.float64)
    ref16 = autograd_of(lambda x, s_: orc.newton_schulz(x.float(), s_), torch.float32)
    saved, U = bw.ns_forward_saved(G.cuda(), 5 if steps is None else steps, steps is not None, False)
    got = bw.ns_backward(saved, dU.cuda()).double().cpu()
    bw.check_status(torch.device("cuda", 0))
    # the recomputed forward uses the kernels' folded arithmetic
    assert orc.rel_fro(U.float().cpu(), orc.newton_schulz_folded(G, steps)) < 3e-2
    assert orc.rel_fro(U.float().cpu(), orc.newton_schulz(G, steps)) < 6e-2
    err_kernel, err_ref = orc.rel_fro(got, ref64), orc.rel_fro(ref16, ref64)
    assert err_kernel <= 1.5 * err_ref + 2e-2, (err_kernel, err_ref)
    assert orc.cosine(got, ref64) >= 0.98


@pytest.mark.parametrize("shape,steps,dtype", [((3, 64, 64), None, torch.float32), ((2, 128, 64), 3, BF16),
                                               ((2, 192, 384), 0, torch.float32)])
def test_newton_schulz_sub_op_is_differentiable(lb, shape, steps, dtype):
    """`zeropower_via_newtonschulz5` under autograd (the reference's function is plain PyTorch, hence differentiable):
    the value equals the plain call's bit for bit and the gradient is the backward helper's."""
    from lact_b200 import backward as bw
    g = torch.Generator().manual_seed(17)
    G = torch.randn(*shape, generator=g).to(dtype).cuda()
    dU = torch.randn(*shape, generator=g).cuda()
    plain = lb.zeropower_via_newtonschulz5(G, steps)
    Gl = G.clone().requires_grad_(True)
    U = lb.zeropower_via_newtonschulz5(Gl, steps)
    assert U.dtype == BF16 and torch.equal(U, plain)
    (U.float() * dU).sum().backward()
    saved, _ = bw.ns_forward_saved(G, 5 if steps is None else steps, steps is not None, False)
    want = bw.ns_backward(saved, dU.to(BF16).float())
    lb.synchronize_and_check()
    assert Gl.grad is not None and Gl.grad.dtype == dtype and torch.isfinite(Gl.grad.float()).all()
    assert torch.equal(Gl.grad.float(), want.to(dtype).float())


@pytest.mark.parametrize("shapes,steps", [
    ([(3, 64, 64), (2, 64, 128)], None),          # 64-wide tiles; square + wide
    ([(4, 256, 128), (4, 128, 128)], None),        # 128-wide tiles; tall + square (the [w0; w2] / w1 pairing)
    ([(20, 768, 384), (20, 384, 384)], None),      # 192-wide tiles, enough work for them
    ([(2, 384, 768)], 3),                          # one group, constant coefficients, 3 iterations
])
def test_newton_schulz_backward_fused_launch(lb, shapes, steps):
    """All iterations of one or two groups in one cooperative launch: against the launch-per-product path on the
    same kept iterates (same operands and roundings except the last gradient, which the fused kernel leaves in bf16
    before the normalisation backward), and against fp64 autograd."""
    from oracle import lact_oracle as orc
    from lact_b200 import backward as bw
    g = torch.Generator().manual_seed(11)
    Gs = [torch.randn(*sh, generator=g) for sh in shapes]
    dUs = [torch.randn(*sh, generator=g) for sh in shapes]
    saved = [bw.ns_forward_saved(G.cuda(), 5 if steps is None else steps, steps is not None, False)[0] for G in Gs]
    from lact_b200 import _lib as LL
    before = LL.launch_count()
    fused = bw.ns_backward_groups(saved, [d.cuda() for d in dUs])
    launches = LL.launch_count() - before
    bw.check_status(torch.device("cuda", 0))
    # one cooperative launch + two small normalisation kernels per group (the launch-per-product path needs
    # three launches per iteration and group)
    assert launches == 1 + 2 * len(shapes), launches
    for sv, G, dU, got in zip(saved, Gs, dUs, fused):
        plain = bw.ns_backward(sv, dU.cuda())
        assert torch.isfinite(got).all()
        assert orc.rel_fro(got.double().cpu(), plain.double().cpu()) <= 1e-2
        if G.shape[1] * G.shape[2] <= 256 * 128:
            Gl = G.to(BF16).double().clone().requires_grad_(True)
            (orc.newton_schulz_f64(Gl, steps) * dU.double()).sum().backward()
            assert orc.cosine(got.double().cpu(), Gl.grad) >= 0.98
    bw.check_status(torch.device("cuda", 0))


def test_llm_backward_with_muon_first_chunks(lb):
    """Muon on: gradients of the tokens that see at most one Newton-Schulz step are compared with
    autograd through the oracle (loose band: the iteration's own bf16 noise, see the forward tests)."""
    from oracle import lact_oracle as orc
    B, L, D, H, C = 2, 256, 64, 64, 128
    inp = orc.make_inputs(B, L, D, H, seed=23)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(5)).to(BF16)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.block_causal_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=True, momentum=m)
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.block_causal_lact_swiglu(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=True, momentum=m)
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, True, dO)
    o, g = _grads_cuda(inp, cu_fn, True, dO)
    for n in ("q", "k", "v", "w0", "w1", "w2", "lr0", "lr1", "lr2"):   # measured: cosine >= 0.9975, rel_fro <= 0.072
        a, b = g[n].float().cpu(), g_ref[n].float()
        assert torch.isfinite(a).all(), n
        assert orc.cosine(a, b) >= 0.995, (n, orc.cosine(a, b))
        assert orc.rel_fro(a, b) <= 0.14, (n, orc.rel_fro(a, b))
    # the fused signature against the oracle with the kernels' own rounding model of the iteration: tighter
    # (measured: cosine >= 0.9994, rel_fro <= 0.035)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.block_causal_lact_swiglu_fused(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=True, momentum=m, ns=orc.newton_schulz_folded)
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=C, use_muon=True, momentum=m)
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, True, dO)
    o, g = _grads_cuda(inp, cu_fn, True, dO)
    for n in ("q", "k", "v", "w0", "w1", "w2", "lr0", "lr1", "lr2"):
        a, b = g[n].float().cpu(), g_ref[n].float()
        assert orc.cosine(a, b) >= 0.998, (n, orc.cosine(a, b))
        assert orc.rel_fro(a, b) <= 0.07, (n, orc.rel_fro(a, b))


@pytest.mark.parametrize("iters", [1, 2])
def test_muon_backward_pins_every_weight_path(lb, iters):
    """Muon on with ONE or TWO Newton-Schulz iterations (the AR driver's `num_moun_iters`, constant coefficients):
    the iteration then amplifies bf16 noise little, so each of the nine gradients -- in particular dW0, dW1 and dW2,
    which reach the loss through three separate Newton-Schulz / renorm paths -- is held to a tight band against
    autograd through the oracle run with the kernels' rounding model of the iteration."""
    from oracle import lact_oracle as orc
    B, L, D, H, mb = 2, 384, 64, 128, 128
    inp = orc.make_inputs(B, L, D, H, seed=31)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(6)).to(BF16)
    kw = dict(mini_batch_size=mb, update_every=mb, use_moun=True, num_moun_iters=iters)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.ar_mini_batch(
        w0, w1, w2, q, k, v, l0, l1, l2, 1.0, ns=orc.newton_schulz_folded, **kw)[0]
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.ar_fast_weight_swish_glu_weight_norm_mini_batch(
        w0, w1, w2, q, k, v, l0, l1, l2, 1.0, **kw)[0]
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, False, dO)
    o, g = _grads_cuda(inp, cu_fn, False, dO)
    assert orc.rel_max(o.float().cpu(), o_ref.float()) <= 3e-2
    for n in NAMES:
        a, b = g[n].float().cpu(), g_ref[n].float()
        assert torch.isfinite(a).all(), n
        rm, cs = orc.rel_max(a, b), orc.cosine(a, b)
        assert cs >= 0.998 and rm <= 5e-2, f"grad {n} ({iters} iterations): rel_max={rm:.3e} cos={cs:.6f}"


def test_muon_and_momentum_backward_tight(lb):
    """Three updates with momentum AND one Newton-Schulz iteration each (the AR driver with momentum): the momentum
    chain's gradient (dbeta through the carried state, the share passed to the previous update) next to the iteration's
    backward, every gradient including the momentum gate's against the oracle with the kernels' rounding model."""
    from oracle import lact_oracle as orc
    B, L, D, H, mb = 2, 512, 64, 128, 128
    inp = orc.make_inputs(B, L, D, H, seed=37)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(9)).to(BF16)
    kw = dict(mini_batch_size=mb, update_every=mb, use_moun=True, num_moun_iters=1, use_momentum=True)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.ar_mini_batch(
        w0, w1, w2, q, k, v, l0, l1, l2, 1.0, fw_momentum=m, ns=orc.newton_schulz_folded, **kw)[0]
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum(
        w0, w1, w2, q, k, v, l0, l1, l2, 1.0, fw_momentum=m, **kw)[0]
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, True, dO)
    o, g = _grads_cuda(inp, cu_fn, True, dO)
    assert orc.rel_max(o.float().cpu(), o_ref.float()) <= 3e-2
    for n in list(NAMES) + ["momentum"]:
        a, b = g[n].float().cpu(), g_ref[n].float()
        assert torch.isfinite(a).all(), n
        rm, cs = orc.rel_max(a, b), orc.cosine(a, b)
        assert cs >= 0.995 and rm <= (0.12 if n == "momentum" else 6e-2), f"grad {n}: rel_max={rm:.3e} cos={cs:.6f}"


@pytest.mark.parametrize("steps", [0, 2])
def test_nvs_operator_list_backward(lb, steps):
    """The NVS driver (transposed weight layout, Gram matrix on the other side for square matrices, constant
    coefficients, target norms detached, one update on the input tokens and one apply on all tokens): gradients against
    autograd through the oracle's restatement of lact_nvs/lact_ttt.py:70-147.  `steps = 0` still divides the gradient
    by its Frobenius norm (the normalisation backward alone); two iterations add the iteration's backward."""
    from oracle import lact_oracle as orc
    B, L, D, H = 2, 384, 64, 64
    inp = orc.make_inputs(B, L, D, H, seed=41)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(3)).to(BF16)
    order = [(0, 256, True, False), (0, 384, False, True)]
    t = lambda w: w.transpose(1, 2)
    ref_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: orc.nvs_mini_batch_apply(
        t(w0), t(w1), t(w2), q, k, v, l0, l1, l2, order, muon_update_steps=steps)[0]
    cu_fn = lambda w0, w1, w2, q, k, v, l0, l1, l2, m: lb.fast_weight_swish_glu_weight_norm_mini_batch_apply(
        t(w0), t(w1), t(w2), q, k, v, l0, l1, l2, [lb.TTTOperator(*op) for op in order], muon_update_steps=steps)[0]
    o_ref, g_ref = _grads_oracle(orc, inp, ref_fn, False, dO)
    o, g = _grads_cuda(inp, cu_fn, False, dO)
    assert orc.rel_max(o.float().cpu(), o_ref.float()) <= 3e-2
    for n in NAMES:
        a, b = g[n].float().cpu(), g_ref[n].float()
        assert torch.isfinite(a).all(), n
        rm, cs = orc.rel_max(a, b), orc.cosine(a, b)
        assert cs >= 0.997 and rm <= 6e-2, f"grad {n} ({steps} iterations): rel_max={rm:.3e} cos={cs:.6f}"


def test_compiled_caller_sees_one_operator(lb):
    """A caller wrapped in torch.compile (as the reference's layers are) traces through the public
    function without a graph break (fullgraph=True) and gets the eager results, forward and backward."""
    from oracle import lact_oracle as orc
    B, L, D, H, C = 2, 512, 64, 64, 128
    inp = orc.make_inputs(B, L, D, H, seed=27)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].to(BF16)
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(9)).to(BF16)

    def layer(w0, w1, w2, q, k, v, l0, l1, l2, m):
        o = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(w0, w1, w2, q * 1.0, k, v, l0, l1, l2, chunk_size=C,
                                                                     use_muon=True, momentum=m)
        return o * 2.0

    compiled = torch.compile(layer, backend="aot_eager", fullgraph=True)
    o_e, g_e = _grads_cuda(inp, layer, True, dO)
    o_c, g_c = _grads_cuda(inp, compiled, True, dO)
    assert torch.equal(o_e, o_c)
    for n in list(NAMES) + ["momentum"]:
        assert torch.equal(g_e[n], g_c[n]), n
    with torch.no_grad():
        c = {k: v.cuda() for k, v in inp.items() if torch.is_tensor(v)}
        assert torch.equal(compiled(*[c[n] for n in NAMES], c["momentum"]), layer(*[c[n] for n in NAMES], c["momentum"]))
