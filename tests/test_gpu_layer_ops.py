"""Layer prologue on the GPU against the CPU oracle (which is pinned bit-exact to the reference's own outputs,
tests/test_oracle_golden.py) and against the reference fixtures directly."""
import os

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


def _ulp_report(got: torch.Tensor, ref: torch.Tensor):
    """(fraction of elements that differ, largest difference in bf16 ulps of the reference value)."""
    g, r = got.float().cpu(), ref.float().cpu()
    diff = (g - r).abs()
    ulp = torch.maximum(r.abs(), torch.full_like(r, 2.0 ** -126)).log2().floor().exp2() * 2.0 ** -7
    return float((diff > 0).float().mean()), float((diff / ulp).max())


def _check(got, ref, what):
    frac, worst = _ulp_report(got, ref)
    # expf and the order of the fp32 row sum may move a value across a bf16 rounding boundary: at most one ulp of
    # the element (two where the row norm itself moved by one ulp), and only for a small share of the elements
    assert worst <= 2.0 and frac <= 0.02, f"{what}: {frac:.4%} of elements differ, worst {worst} ulp"


@pytest.mark.parametrize("b,s,n_h,d,v_silu", [(2, 37, 4, 64, True), (1, 130, 2, 384, False), (3, 16, 3, 192, True),
                                              (1, 5, 1, 1024, True), (2, 9, 6, 8, True)])
def test_qkv_prologue_against_oracle(lb, orc, b, s, n_h, d, v_silu):
    from lact_b200 import layer_ops
    g = torch.Generator().manual_seed(7)
    xq, xk, xv = (torch.randn(b, s, n_h * d, generator=g).to(BF16) * 1.5 for _ in range(3))
    rq, rk, rv = orc.qkv_prologue(xq, xk, xv, n_h, True, v_silu)
    q, k, v = layer_ops.qkv_prologue(xq.cuda(), xk.cuda(), xv.cuda(), n_h, qkv_silu=True, no_v_silu=not v_silu)
    assert q.shape == rq.shape and q.dtype == BF16 and q.is_contiguous()
    _check(q, rq, "q"); _check(k, rk, "k"); _check(v, rv, "v")
    # without SiLU the values of v pass through untouched and q, k are only normalised
    rq, rk, rv = orc.qkv_prologue(xq, xk, xv, n_h, False, v_silu)
    q, k, v = layer_ops.qkv_prologue(xq.cuda(), xk.cuda(), xv.cuda(), n_h, qkv_silu=False)
    _check(q, rq, "q (no silu)"); _check(k, rk, "k (no silu)")
    assert torch.equal(v.cpu(), rv)


def test_qkv_prologue_reference_fixtures_and_fused_projection_views(lb, orc):
    from lact_b200 import layer_ops
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    for name, case in blob.items():
        if name.startswith(("lr_", "out_", "rope_")):
            continue
        sp = case["spec"]
        g = torch.Generator().manual_seed(sp["seed"])
        xq, xk, xv = (torch.randn(sp["b"], sp["s"], sp["n_h"] * sp["d"], generator=g).to(BF16) * 1.5 for _ in range(3))
        # the three projections as column blocks of one fused [b, s, 3 n_h d] tensor (strided views)
        fused = torch.cat([xq, xk, xv], dim=-1).cuda()
        nd = sp["n_h"] * sp["d"]
        vq, vk, vv = fused[..., :nd], fused[..., nd:2 * nd], fused[..., 2 * nd:]
        assert not vq.is_contiguous()
        q, k, v = layer_ops.qkv_prologue(vq, vk, vv, sp["n_h"], no_v_silu=not sp["v_silu"])
        _check(q, case["q"], name + " q"); _check(k, case["k"], name + " k"); _check(v, case["v"], name + " v")


def test_qkv_prologue_rejects_bad_arguments(lb):
    from lact_b200 import layer_ops
    x = torch.zeros(1, 4, 24, dtype=BF16, device="cuda")
    with pytest.raises(ValueError):
        layer_ops.qkv_prologue(x, x, x, 2)          # d = 12 is not a multiple of 8
    with pytest.raises(ValueError):
        layer_ops.qkv_prologue(x.cpu(), x.cpu(), x.cpu(), 3)
    with pytest.raises(AssertionError):
        layer_ops.qkv_prologue(x.float(), x.float(), x.float(), 3)


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
def test_lr_prologue_against_oracle_and_reference_fixtures(lb, orc, dtype):
    from lact_b200 import layer_ops
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    for name, case in blob.items():
        if not name.startswith("lr_"):
            continue
        sp = case["spec"]
        g = torch.Generator().manual_seed(sp["seed"])
        proj = (torch.randn(sp["b"], sp["s"], sp["n_h"] * 3, generator=g) * 2.0).to(BF16).to(dtype)
        mlogit = (torch.randn(sp["b"], sp["s"], sp["n_h"], generator=g) * 2.0).to(BF16).to(dtype)
        ref = orc.lr_prologue(proj, sp["n_h"], sp["base_lr"], mlogit)
        got = layer_ops.lr_prologue(proj.cuda(), sp["n_h"], sp["base_lr"], mlogit.cuda())
        for r, x, what in zip(ref, got, ("lr0", "lr1", "lr2", "momentum")):
            assert x.shape == r.shape and x.dtype == torch.float32
            # fp32 softplus / sigmoid: a few ulp of expf / log1pf; the bf16-rounded sigmoid may move by one bf16 ulp
            tol = 2.0 ** -7 if (what == "momentum" and dtype == BF16) else 2e-6
            assert float(((x.cpu() - r).abs() / r.abs().clamp_min(1e-30)).max()) <= tol, (name, what)
        if dtype == BF16:  # the bf16 run is the reference fixture's own case
            assert float((got[0].cpu() - case["lr0"]).abs().max()) <= 2e-6 * float(case["lr0"].abs().max())
            assert float((got[3].cpu() != case["momentum"]).float().mean()) <= 0.01
    no_mom = layer_ops.lr_prologue(torch.zeros(1, 3, 6, device="cuda"), 2, 1e-2)
    assert no_mom[3] is None and abs(float(no_mom[0][0, 0, 0]) - 1e-2) < 1e-6  # softplus(inv_softplus(base_lr)) = base_lr


@pytest.mark.parametrize("b,s,n_h,d", [(2, 37, 4, 64), (1, 50, 2, 384), (2, 9, 3, 8), (1, 3, 1, 1024)])
def test_out_epilogue_against_oracle(lb, orc, b, s, n_h, d):
    from lact_b200 import layer_ops
    g = torch.Generator().manual_seed(11)
    fw_x = (torch.randn(b * n_h, s, d, generator=g) * 2.0).to(BF16)
    weight = 1.0 + 0.1 * torch.randn(d, generator=g)
    sproj = (torch.randn(b, s, n_h * d, generator=g) * 1.5).to(BF16)
    o_attn = torch.randn(b, s, n_h * d, generator=g).to(BF16)
    for use_gate, use_res in ((True, True), (False, True), (True, False), (False, False)):
        ref = orc.out_epilogue(fw_x, weight, n_h, sproj if use_gate else None, o_attn if use_res else None)
        got = layer_ops.out_epilogue(fw_x.cuda(), weight.cuda(), n_h, sproj.cuda() if use_gate else None,
                                     o_attn.cuda() if use_res else None)
        assert got.shape == ref.shape and got.dtype == BF16
        # chained bf16 roundings: a one-ulp move of the normalised value or of the gate moves the result by an ulp or two
        frac, worst = _ulp_report(got, ref)
        assert worst <= 4.0 and frac <= 0.03, (use_gate, use_res, frac, worst)


def test_out_epilogue_reference_fixtures(lb, orc):
    from lact_b200 import layer_ops
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    for name, case in blob.items():
        if not name.startswith("out_"):
            continue
        sp = case["spec"]
        b, s, n_h, d = sp["b"], sp["s"], sp["n_h"], sp["d"]
        g = torch.Generator().manual_seed(sp["seed"])
        fw_x = (torch.randn(b * n_h, s, d, generator=g) * 2.0).to(BF16)
        weight = 1.0 + 0.1 * torch.randn(d, generator=g)
        sproj = (torch.randn(b, s, n_h * d, generator=g) * 1.5).to(BF16)
        o_attn = torch.randn(b, s, n_h * d, generator=g).to(BF16)
        got = layer_ops.out_epilogue(fw_x.cuda(), weight.cuda(), n_h, sproj.cuda(), o_attn.cuda())
        frac, worst = _ulp_report(got, case["out"])
        assert worst <= 4.0 and frac <= 0.03, (name, frac, worst)



@pytest.mark.parametrize("b,s,n_h,d,hd,off", [(2, 37, 4, 64, 64, 0), (1, 130, 2, 384, 128, 5), (2, 16, 2, 128, 32, 3),
                                              (1, 9, 1, 512, 256, 0), (1, 7, 1, 1024, 512, 2), (1, 6, 2, 256, 128, 1)])
def test_qkv_prologue_with_rotary_embedding(lb, orc, b, s, n_h, d, hd, off):
    """Rotary embedding of fast q, k fused into the pass (layer_lact_swiglu.py:417-446): against the oracle's fused
    (fp32, single rounding) arithmetic within the band of the plain pass, and against the restatement of fla's own
    PyTorch rotation (three bf16 roundings) within two more ulps at the inputs' scale; v is untouched by the rotation."""
    from lact_b200 import layer_ops
    g = torch.Generator().manual_seed(11)
    xq, xk, xv = (torch.randn(b, s, n_h * d, generator=g).to(BF16) * 1.5 for _ in range(3))
    cos, sin = orc.rotary_tables(hd, off + s + 3)
    dcos, dsin = layer_ops.rotary_tables(hd, off + s + 3, device="cuda")
    assert torch.equal(dcos.cpu(), cos) or float((dcos.cpu().float() - cos.float()).abs().max()) <= 2.0 ** -8
    q, k, v = layer_ops.qkv_prologue(xq.cuda(), xk.cuda(), xv.cuda(), n_h, rotary=(cos.cuda(), sin.cuda(), hd),
                                     seqlen_offset=off)
    fq, fk, fv = orc.qkv_prologue_rope(xq, xk, xv, n_h, hd, cos, sin, off, policy="fused")
    rq, rk, _ = orc.qkv_prologue_rope(xq, xk, xv, n_h, hd, cos, sin, off, policy="ref")
    for got, fused, ref, what in ((q, fq, rq, "q"), (k, fk, rk, "k")):
        gf = got.float().cpu()
        # a one-ulp difference of an l2-normed input (fast exponential, order of the row sum) rotates into both
        # partners: measured against the scale of the row (|x| <= 1), not of the single element
        scale = 2.0 ** -8
        assert float((gf - fused.float()).abs().max()) <= 2 * scale, what
        assert float(((gf - fused.float()).abs() > 0).float().mean()) <= 0.05, what
        assert float((gf - ref.float()).abs().max()) <= 3 * scale, what
    _check(v, fv, "v")
    # the first token at offset 0 is not rotated (cos = 1, sin = 0)
    if off == 0:
        pq, _, _ = layer_ops.qkv_prologue(xq.cuda(), xk.cuda(), xv.cuda(), n_h)
        assert torch.equal(q[:, 0], pq[:, 0])
    # argument errors: head size that does not tile the fast-weight head, positions beyond the table
    with pytest.raises(ValueError):
        layer_ops.qkv_prologue(xq.cuda(), xk.cuda(), xv.cuda(), n_h, rotary=(cos.cuda(), sin.cuda(), hd),
                               seqlen_offset=off + 10)


def test_layer_passes_are_differentiable(lb, orc):
    """Gradients of the three layer passes against autograd through the oracle's formulas in fp32."""
    from lact_b200 import layer_ops
    b, s, n_h, d, hd = 2, 24, 2, 128, 64
    g = torch.Generator().manual_seed(12)
    xs = [(torch.randn(b, s, n_h * d, generator=g) * 1.5).to(BF16) for _ in range(3)]
    cos, sin = orc.rotary_tables(hd, s)
    dO = [torch.randn(b * n_h, s, d, generator=g) for _ in range(3)]
    # reference gradients: fp32 autograd through the oracle (fused rounding policy has no roundings in fp32)
    leaves = [t.float().clone().requires_grad_(True) for t in xs]
    ref = torch.autograd.grad(orc.qkv_prologue_rope(*leaves, n_h, hd, cos.float(), sin.float(), 0, policy="fused"), leaves, dO)
    cl = [t.cuda().clone().requires_grad_(True) for t in xs]
    q, k, v = layer_ops.qkv_prologue(*cl, n_h, rotary=(cos.cuda(), sin.cuda(), hd))
    torch.autograd.backward([q, k, v], [t.cuda().to(BF16) for t in dO])
    for got, want, what in zip(cl, ref, ("dxq", "dxk", "dxv")):
        assert got.grad is not None and got.grad.dtype == BF16
        assert orc.rel_max(got.grad.float().cpu(), want) <= 2e-2 and orc.cosine(got.grad.float().cpu(), want) >= 0.999, what
    # learning rates / momentum
    proj = (torch.randn(b, s, n_h * 3, generator=g) * 2).to(BF16)
    logit = (torch.randn(b, s, n_h, generator=g) * 2).to(BF16)
    gl = [torch.randn(b * n_h, s, 1, generator=g) for _ in range(4)]
    pl, ml = proj.float().clone().requires_grad_(True), logit.float().clone().requires_grad_(True)
    ref = torch.autograd.grad(orc.lr_prologue(pl, n_h, 1e-2, ml), [pl, ml], gl)
    cp, cm = proj.cuda().clone().requires_grad_(True), logit.cuda().clone().requires_grad_(True)
    o4 = layer_ops.lr_prologue(cp, n_h, 1e-2, cm)
    torch.autograd.backward(list(o4), [t.cuda() for t in gl])
    assert orc.rel_max(cp.grad.float().cpu(), ref[0]) <= 1e-2 and orc.rel_max(cm.grad.float().cpu(), ref[1]) <= 1e-2
    # output epilogue
    fw_x = (torch.randn(b * n_h, s, d, generator=g) * 2).to(BF16)
    w = 1.0 + 0.1 * torch.randn(d, generator=g)
    sp, oa = torch.randn(b, s, n_h * d, generator=g).to(BF16), torch.randn(b, s, n_h * d, generator=g).to(BF16)
    gout = torch.randn(b, s, n_h * d, generator=g)
    L4 = [t.float().clone().requires_grad_(True) for t in (fw_x, w, sp, oa)]
    ref = torch.autograd.grad(orc.out_epilogue(L4[0], L4[1], n_h, L4[2], L4[3]), L4, gout)
    C4 = [t.cuda().clone().requires_grad_(True) for t in (fw_x, w, sp, oa)]
    out = layer_ops.out_epilogue(C4[0], C4[1], n_h, C4[2], C4[3])
    out.backward(gout.cuda().to(out.dtype))
    for got, want, what in zip(C4, ref, ("d fw_x", "d weight", "d scale_proj", "d o")):
        assert got.grad is not None, what
        assert orc.rel_max(got.grad.float().cpu(), want) <= 2e-2 and orc.cosine(got.grad.float().cpu(), want) >= 0.999, what


def test_rotary_prologue_with_packed_sequences(lb, orc):
    """cu_seqlens: positions restart at every sequence start (layer_lact_swiglu.py:434), forward and gradients."""
    from lact_b200 import layer_ops as lo
    b, s, n_h, d, hd = 1, 300, 2, 128, 64
    cu = torch.tensor([0, 70, 71, 200, 300], dtype=torch.int32)
    g = torch.Generator().manual_seed(21)
    xs = [torch.randn(b, s, n_h * d, generator=g).to(BF16) for _ in range(3)]
    dz = [torch.randn(b * n_h, s, d, generator=g).to(BF16) for _ in range(3)]
    cos, sin = orc.rotary_tables(hd, s)
    leaves = [x.float().clone().requires_grad_(True) for x in xs]
    ref = orc.qkv_prologue_rope(*leaves, n_h, hd, cos, sin, policy="fused", cu_seqlens=cu)
    sum((r.float() * z.float()).sum() for r, z in zip(ref, dz)).backward()
    cl = [x.cuda().clone().requires_grad_(True) for x in xs]
    got = lo.qkv_prologue(*cl, n_h, rotary=(cos.cuda(), sin.cuda(), hd), cu_seqlens=cu.cuda())
    torch.autograd.backward(got, [z.cuda() for z in dz])
    for a, r in zip(got, ref):
        assert orc.rel_max(a.detach().float().cpu(), r.detach().float()) <= 2e-2
    for a, r in zip(cl, leaves):
        assert orc.rel_max(a.grad.float().cpu(), r.grad) <= 3e-2 and orc.cosine(a.grad.float().cpu(), r.grad) >= 0.999
    # without cu_seqlens the later sequences get different positions: the outputs must differ there
    plain = lo.qkv_prologue(*[c.detach() for c in cl], n_h, rotary=(cos.cuda(), sin.cuda(), hd))
    assert not torch.equal(plain[0][:, 100:], got[0][:, 100:].detach())
    assert torch.equal(plain[0][:, :70], got[0][:, :70].detach())


def test_layer_passes_against_the_fla_kernels_when_they_run(lb, orc):
    """The library kernels the reference layer itself calls (flash-linear-attention's Triton RotaryEmbedding and
    RMSNorm, lact_llm/lact_model/layer_lact_swiglu.py:170, 242, 429, 557), run on this GPU on the same inputs: the
    rotary prologue after the reference's own SiLU / l2_norm arithmetic, and the per-head RMSNorm of the output
    epilogue.  Skipped where the package or its Triton backend is not usable."""
    fla_modules = pytest.importorskip("fla.modules")
    import torch.nn.functional as F
    from lact_b200 import layer_ops as lo
    b, s, n_h, d, hd = 2, 300, 2, 384, 128
    g = torch.Generator().manual_seed(51)
    xq, xk, xv = ((torch.randn(b, s, n_h * d, generator=g) * 0.8).to(BF16).cuda() for _ in range(3))
    try:
        rot = fla_modules.RotaryEmbedding(dim=hd, base=500000.0).cuda()
        heads = lambda t: t.reshape(b, s, n_h, d).permute(0, 2, 1, 3).reshape(b * n_h, s, d)
        l2n = lambda x: (x / (x.norm(dim=-1, keepdim=True) + 1e-5)).type(x.dtype)   # ttt_operation.py:19-26
        fq, fk = l2n(heads(F.silu(xq))), l2n(heads(F.silu(xk)))
        merge = lambda t: t.reshape(b, n_h, s, d).permute(0, 2, 1, 3).reshape(b, s, (n_h * d) // hd, hd)
        rq, rk = rot(merge(fq), merge(fk), seqlen_offset=0, max_seqlen=s)
        back = lambda t: heads(t.reshape(b, s, n_h * d))
        want_q, want_k = back(rq), back(rk)
        norm = fla_modules.RMSNorm(d, elementwise_affine=True, eps=1e-5).cuda()
        with torch.no_grad():
            norm.weight.copy_(1.0 + 0.1 * torch.randn(d, generator=g).cuda())
        fw = (torch.randn(b * n_h, s, d, generator=g) * 0.5).to(BF16).cuda()
        want_n = norm(fw).detach()
        torch.cuda.synchronize()
    except Exception as e:   # no usable Triton backend for this GPU in the installed package
        pytest.skip(f"fla kernels did not run here: {type(e).__name__}: {str(e)[:120]}")
    cos, sin = lo.rotary_tables(hd, s, device="cuda")
    got_q, got_k, _ = lo.qkv_prologue(xq, xk, xv, n_h, rotary=(cos, sin, hd))
    got_n = lo.out_epilogue(fw, norm.weight.detach(), n_h)
    lb.synchronize_and_check()
    # fla's rotary kernel contracts x cos - y sin differently from its own PyTorch restatement (which the oracle and
    # this package follow bit for bit): where the two products cancel, the results differ by several ulps OF THE TINY
    # RESULT, so the rotation is held to one bf16 ulp at the scale of the operands instead (2^-8 of the largest value)
    for name, got, want in (("q", got_q, want_q), ("k", got_k, want_k)):
        frac, _ = _ulp_report(got, want)
        worst = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert frac <= 0.02 and worst <= 2.0 ** -8, f"rotary {name} vs fla: {frac:.4%} differ, worst {worst:.2e} of the maximum"
    _check(got_n, want_n.reshape(b, n_h, s, d).permute(0, 2, 1, 3).reshape(b, s, n_h * d), "RMSNorm vs fla")
