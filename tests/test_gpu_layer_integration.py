"""The whole hybrid layer built from this package's operators -- projections (plain torch.nn.functional.linear), the
q / k / v prologue with rotary embedding, the learning-rate prologue, the chunk recurrence (fused post-norm signature,
Muon + momentum), sliding-window attention on the same projections, and the output epilogue -- against the same
composition of the CPU oracle's restatements (lact_llm/lact_model/layer_lact_swiglu.py:386-568 is the reference's
sequence of steps), forward values and, with Muon off, gradients of every parameter; then two layers stacked, a
backward through all of them, and the status ring read at the end."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    import lact_b200
    from lact_b200 import layer_ops
    from oracle import lact_oracle as orc
    return lact_b200, layer_ops, orc


def make_params(hidden, n_heads, attn_heads, seed):
    g = torch.Generator().manual_seed(seed)
    d = hidden // n_heads
    rn = lambda *s, scale=1.0: torch.randn(*s, generator=g) * scale
    return dict(
        wqkv=rn(3 * hidden, hidden, scale=hidden ** -0.5).to(BF16),        # one fused projection
        wlr=rn(3 * n_heads, hidden, scale=hidden ** -0.5).to(BF16),
        wmom=rn(n_heads, hidden, scale=hidden ** -0.5).to(BF16),
        wgate=rn(hidden, hidden, scale=hidden ** -0.5).to(BF16),
        norm=1.0 + 0.1 * rn(d),
        w0=rn(n_heads, d, d, scale=d ** -0.5), w1=rn(n_heads, d, d, scale=d ** -0.5), w2=rn(n_heads, d, d, scale=d ** -0.5),
    )


def layer(x, p, cfg, ops):
    """One hybrid layer.  `ops` supplies the six operators (this package's, or the oracle's)."""
    b, s, hidden = x.shape
    n_h, a_h, chunk, window, muon = cfg
    qkv = F.linear(x, p["wqkv"])
    xq, xk, xv = qkv.chunk(3, dim=-1)
    cos, sin = ops["tables"](hidden // a_h, s)
    fq, fk, fv = ops["qkv"](xq, xk, xv, n_h, hidden // a_h, cos, sin)
    lr0, lr1, lr2, mom = ops["lr"](F.linear(x, p["wlr"]), n_h, 0.01, F.linear(x, p["wmom"]))
    rep = lambda w: w.repeat(b, 1, 1)
    fw = ops["ttt"](rep(p["w0"]), rep(p["w1"]), rep(p["w2"]), fq, fk, fv, lr0, lr1, lr2, chunk, muon, mom)
    hd = hidden // a_h
    att = ops["swa"](xq.reshape(b, s, a_h, hd), xk.reshape(b, s, a_h, hd), xv.reshape(b, s, a_h, hd), window)
    return ops["out"](fw, p["norm"], n_h, F.linear(x, p["wgate"]), att.reshape(b, s, hidden).to(x.dtype))


def cuda_ops(lb, lo):
    return dict(
        tables=lambda hd, n: lo.rotary_tables(hd, n, device="cuda"),
        qkv=lambda xq, xk, xv, n_h, hd, cos, sin: lo.qkv_prologue(xq, xk, xv, n_h, rotary=(cos, sin, hd)),
        lr=lo.lr_prologue,
        ttt=lambda w0, w1, w2, q, k, v, l0, l1, l2, chunk, muon, mom: lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
            w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=chunk, use_muon=muon, momentum=mom),
        swa=lo.sliding_window_attention,
        out=lo.out_epilogue,
    )


def oracle_ops(orc):
    return dict(
        tables=lambda hd, n: orc.rotary_tables(hd, n),
        qkv=lambda xq, xk, xv, n_h, hd, cos, sin: orc.qkv_prologue_rope(xq, xk, xv, n_h, hd, cos, sin, policy="fused"),
        lr=orc.lr_prologue,
        ttt=lambda w0, w1, w2, q, k, v, l0, l1, l2, chunk, muon, mom: orc.block_causal_lact_swiglu_fused(
            w0, w1, w2, q, k, v, l0, l1, l2, chunk_size=chunk, use_muon=muon, momentum=mom),
        swa=lambda q, k, v, w: orc.sliding_window_attention(q, k, v, w),
        out=lambda fw, w, n_h, gate, o: orc.out_epilogue(fw, w, n_h, gate, o),
    )


def test_hybrid_layer_forward_and_gradients_muon_off(mods):
    lb, lo, orc = mods
    b, s, hidden, n_h, a_h = 2, 512, 256, 2, 4          # fast-weight heads of 128, attention heads of 64
    cfg = (n_h, a_h, 128, 96, False)
    p = make_params(hidden, n_h, a_h, seed=1)
    x = (torch.randn(b, s, hidden, generator=torch.Generator().manual_seed(2)) * 0.5).to(BF16)
    dy = torch.randn(b, s, hidden, generator=torch.Generator().manual_seed(3)).to(BF16)
    # oracle: fp32 arithmetic on the same bf16 parameters and input
    pr = {k: v.float().clone().requires_grad_(True) for k, v in p.items()}
    xr = x.float().clone().requires_grad_(True)
    yr = layer(xr, pr, cfg, oracle_ops(orc))
    (yr.float() * dy.float()).sum().backward()
    pc = {k: v.cuda().clone().requires_grad_(True) for k, v in p.items()}
    xc = x.cuda().clone().requires_grad_(True)
    yc = layer(xc, pc, cfg, cuda_ops(lb, lo))
    yc.backward(dy.cuda())
    lb.synchronize_and_check()
    assert yc.dtype == BF16 and yc.shape == (b, s, hidden)
    assert orc.rel_max(yc.detach().float().cpu(), yr.detach().float()) <= 3e-2
    assert orc.cosine(yc.detach().float().cpu(), yr.detach().float()) >= 0.9995
    for name in list(p) + ["x"]:
        got = (xc if name == "x" else pc[name]).grad
        want = (xr if name == "x" else pr[name]).grad
        assert got is not None and torch.isfinite(got.float()).all(), name
        cs = orc.cosine(got.float().cpu(), want.float())
        assert cs >= 0.995, (name, cs)


def test_two_stacked_layers_train_step_with_muon(mods):
    lb, lo, orc = mods
    b, s, hidden, n_h, a_h = 1, 768, 256, 2, 2          # attention heads of 128
    cfg = (n_h, a_h, 256, 300, True)
    ps = [{k: v.cuda().clone().requires_grad_(True) for k, v in make_params(hidden, n_h, a_h, seed=10 + i).items()}
          for i in range(2)]
    x = (torch.randn(b, s, hidden, generator=torch.Generator().manual_seed(4)) * 0.5).to(BF16).cuda().requires_grad_(True)
    ops = cuda_ops(lb, lo)
    outs = []
    for rep in range(2):   # the same step twice: identical results (no state leaks between calls, deterministic kernels)
        for p in ps:
            for t in p.values():
                t.grad = None
        x.grad = None
        h = x
        for p in ps:
            h = (h.float() + layer(h, p, cfg, ops).float()).to(BF16)   # residual connection
        h.float().square().mean().backward()
        outs.append((h.detach().clone(), x.grad.clone(), ps[0]["w1"].grad.clone(), ps[1]["wqkv"].grad.clone()))
    lb.synchronize_and_check()
    for t in outs[0]:
        assert torch.isfinite(t.float()).all()
    for a, b_ in zip(outs[0], outs[1]):
        assert torch.equal(a, b_)


def test_nvs_layer_chain(mods):
    """The novel-view-synthesis block (lact_nvs/lact_ttt.py:204-245): SiLU of the fused q / k / v projection, l2 norm of
    q and k, softplus learning rates (the reference orders the lr projection (lrs, head); the kernel wants (head, lrs):
    the rows of the Linear are permuted once), the operator-list recurrence in the transposed weight layout with
    Muon, RMSNorm of the result and the head merge -- this package's operators against the oracle's, forward."""
    lb, lo, orc = mods
    b, l, hidden, n_h = 2, 640, 256, 2
    d = hidden // n_h
    g = torch.Generator().manual_seed(21)
    rn = lambda *s, scale=1.0: torch.randn(*s, generator=g) * scale
    p = dict(wqkv=rn(3 * hidden, hidden, scale=hidden ** -0.5).to(BF16), wlr=rn(3 * n_h, hidden, scale=hidden ** -0.5),
             norm=1.0 + 0.1 * rn(d), w0=rn(n_h, d, d, scale=d ** -0.5), w1=rn(n_h, d, d, scale=d ** -0.5),
             w2=rn(n_h, d, d, scale=d ** -0.5))
    x = (rn(b, l, hidden) * 0.5).to(BF16)
    order = [(0, 128, False, True), (0, 384, True, False), (384, 512, True, True), (512, 640, False, True)]
    base_lr, steps = 0.01, 5
    # (lrs, head) -> (head, lrs)
    perm = torch.tensor([lrs * n_h + h for h in range(n_h) for lrs in range(3)])

    def chain(x, p, ops, dev):
        xq, xk, xv = F.linear(x, p["wqkv"]).chunk(3, dim=-1)
        fq, fk, fv = ops["qkv"](xq, xk, xv, n_h)
        lr0, lr1, lr2, _ = ops["lr"](F.linear(x.float(), p["wlr"][perm.to(dev)]), n_h, base_lr, None)
        rep = lambda w: w.repeat(b, 1, 1)
        out, *_ = ops["ttt"](rep(p["w0"]), rep(p["w1"]), rep(p["w2"]), fq, fk, fv, lr0, lr1, lr2, order, steps)
        return ops["out"](out, p["norm"], n_h, None, None)

    ref = chain(x, p, dict(qkv=orc.qkv_prologue, lr=orc.lr_prologue,
                           ttt=lambda *a: orc.nvs_mini_batch_apply(*a, nm=orc.Numerics("ref", autocast=True)),
                           out=lambda fw, w, n, gate, o: orc.out_epilogue(fw, w, n, gate, o)), "cpu")
    pc = {k: v.cuda() for k, v in p.items()}
    got = chain(x.cuda(), pc, dict(qkv=lo.qkv_prologue, lr=lo.lr_prologue,
                                   ttt=lb.fast_weight_swish_glu_weight_norm_mini_batch_apply, out=lo.out_epilogue), "cuda")
    lb.synchronize_and_check()
    assert got.shape == (b, 384, hidden) and got.dtype == BF16   # the three apply operators' tokens, in list order
    # the first apply uses the initial weights (exact band); the others carry one or two Newton-Schulz passes
    assert orc.rel_max(got[:, :128].float().cpu(), ref[:, :128].float()) <= 3e-2
    cs, rm = orc.cosine(got.float().cpu(), ref.float()), orc.rel_max(got.float().cpu(), ref.float())
    assert cs >= 0.995 and rm <= 1e-1, (cs, rm)
