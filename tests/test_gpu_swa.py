"""Causal sliding-window attention kernel against the CPU oracle (fp32 softmax attention over the band):
head dimensions 64 and 128, windows smaller / larger than the sequence and not multiples of the tile,
ragged sequence lengths, strided views of a fused projection, a window of one key."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def lo():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    from lact_b200 import layer_ops
    return layer_ops


def _check(lo, q, k, v, window):
    import lact_b200
    from oracle import lact_oracle as orc
    got = lo.sliding_window_attention(q.cuda(), k.cuda(), v.cuda(), window)
    lact_b200.synchronize_and_check()
    ref = orc.sliding_window_attention(q, k, v, window)
    got = got.float().cpu()
    assert torch.isfinite(got).all()
    # bf16 probabilities and bf16 output: a few 2^-9 of the row's largest value
    err = (got - ref).abs().max() / ref.abs().max()
    assert err <= 1.5e-2, float(err)
    assert orc.cosine(got, ref) >= 0.9999


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("l,window", [(1024, 256), (1000, 300), (777, None), (128, 64), (65, 1), (2500, 2048), (640, 129)])
def test_swa_matches_oracle(lo, d, l, window):
    g = torch.Generator().manual_seed(l + d)
    q, k, v = (torch.randn(2, l, 3, d, generator=g).to(BF16) for _ in range(3))
    _check(lo, q, k, v, window)


def test_swa_on_views_of_a_fused_projection(lo):
    """q, k, v as the three slices of one [b, l, 3 * h * d] projection (token stride 3 h d), no copies."""
    import lact_b200
    from oracle import lact_oracle as orc
    b, l, h, d = 2, 512, 4, 128
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(b, l, 3 * h * d, generator=g).to(BF16)
    dev = qkv.cuda()
    qv, kv, vv = (t.reshape(b, l, h, d) for t in dev.chunk(3, dim=-1))
    assert not qv.is_contiguous()
    got = lo.sliding_window_attention(qv, kv, vv, 200)
    lact_b200.synchronize_and_check()
    q, k, v = (t.reshape(b, l, h, d) for t in qkv.chunk(3, dim=-1))
    ref = orc.sliding_window_attention(q, k, v, 200)
    assert (got.float().cpu() - ref).abs().max() / ref.abs().max() <= 1.5e-2


def test_swa_large_scores_and_scale(lo):
    """Scores far from zero (the running maximum changes from tile to tile) and a caller-given scale."""
    import lact_b200
    from oracle import lact_oracle as orc
    g = torch.Generator().manual_seed(5)
    b, l, h, d = 1, 900, 2, 64
    q = (torch.randn(b, l, h, d, generator=g) * 3).to(BF16)
    k = (torch.randn(b, l, h, d, generator=g) * 3).to(BF16)
    v = torch.randn(b, l, h, d, generator=g).to(BF16)
    got = lo.sliding_window_attention(q.cuda(), k.cuda(), v.cuda(), 400, softmax_scale=0.2)
    lact_b200.synchronize_and_check()
    ref = orc.sliding_window_attention(q, k, v, 400, softmax_scale=0.2)
    assert torch.isfinite(got.float()).all()
    assert (got.float().cpu() - ref).abs().max() / ref.abs().max() <= 2e-2


def test_swa_rejects_unsupported_head_dim(lo):
    q = torch.randn(1, 64, 2, 96).to(BF16).cuda()
    with pytest.raises(ValueError):
        lo.sliding_window_attention(q, q, q, 16)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("l,window", [(512, 200), (300, None), (700, 129), (128, 1), (1100, 1024)])
def test_swa_backward_matches_autograd_of_the_oracle(lo, d, l, window):
    """dq, dk, dv against autograd through the oracle's fp32 banded attention on the same bf16 inputs."""
    import lact_b200
    from oracle import lact_oracle as orc
    g = torch.Generator().manual_seed(7 * l + d)
    q, k, v = (torch.randn(2, l, 2, d, generator=g).to(BF16) for _ in range(3))
    dO = torch.randn(2, l, 2, d, generator=g).to(BF16)
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    (orc.sliding_window_attention(*leaves, window) * dO.float()).sum().backward()
    cl = [t.cuda().clone().requires_grad_(True) for t in (q, k, v)]
    o = lo.sliding_window_attention(*cl, window)
    o.backward(dO.cuda())
    lact_b200.synchronize_and_check()
    for name, got, want in zip("qkv", cl, leaves):
        a, b_ = got.grad.float().cpu(), want.grad
        assert torch.isfinite(a).all(), name
        if float(b_.abs().max()) == 0.0:   # a window of one key: the probabilities are constant, dq and dk vanish
            assert float(a.abs().max()) <= 1e-2, name
            continue
        assert orc.rel_max(a, b_) <= 3e-2 and orc.cosine(a, b_) >= 0.9995, (name, orc.rel_max(a, b_), orc.cosine(a, b_))


def test_swa_backward_on_views_and_partial_graph(lo):
    """Strided views of a fused projection as inputs; only q requires grad."""
    import lact_b200
    from oracle import lact_oracle as orc
    b, l, h, d = 1, 384, 3, 128
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(b, l, 3 * h * d, generator=g).to(BF16)
    dO = torch.randn(b, l, h, d, generator=g).to(BF16)
    dev = qkv.cuda().requires_grad_(True)
    qv, kv, vv = (t.reshape(b, l, h, d) for t in dev.chunk(3, dim=-1))
    lo.sliding_window_attention(qv, kv, vv, 100).backward(dO.cuda())
    lact_b200.synchronize_and_check()
    ref = qkv.float().clone().requires_grad_(True)
    rq, rk, rv = (t.reshape(b, l, h, d) for t in ref.chunk(3, dim=-1))
    (orc.sliding_window_attention(rq, rk, rv, 100) * dO.float()).sum().backward()
    assert orc.rel_max(dev.grad.float().cpu(), ref.grad) <= 3e-2
    assert orc.cosine(dev.grad.float().cpu(), ref.grad) >= 0.9995


@pytest.mark.parametrize("window", [None, 150])
def test_swa_packed_sequences_forward_and_backward(lo, window):
    """cu_seqlens: sequences packed into one batch entry; boundaries inside and on tile edges, a one-token sequence."""
    import lact_b200
    from oracle import lact_oracle as orc
    cu = torch.tensor([0, 100, 101, 384, 700, 1000], dtype=torch.int32)
    l, h, d = 1000, 2, 128
    g = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(1, l, h, d, generator=g).to(BF16) for _ in range(3))
    dO = torch.randn(1, l, h, d, generator=g).to(BF16)
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    ref = orc.sliding_window_attention(*leaves, window, cu_seqlens=cu)
    (ref * dO.float()).sum().backward()
    cl = [t.cuda().clone().requires_grad_(True) for t in (q, k, v)]
    o = lo.sliding_window_attention(*cl, window, cu_seqlens=cu.cuda())
    o.backward(dO.cuda())
    lact_b200.synchronize_and_check()
    assert (o.detach().float().cpu() - ref.detach()).abs().max() / ref.detach().abs().max() <= 1.5e-2
    for name, got, want in zip("qkv", cl, leaves):
        a, b_ = got.grad.float().cpu(), want.grad
        assert orc.rel_max(a, b_) <= 3e-2 and orc.cosine(a, b_) >= 0.9995, (name, orc.rel_max(a, b_), orc.cosine(a, b_))
    with pytest.raises(ValueError):
        lo.sliding_window_attention(torch.cat([cl[0]] * 2).detach(), torch.cat([cl[1]] * 2).detach(),
                                    torch.cat([cl[2]] * 2).detach(), window, cu_seqlens=cu.cuda())


@pytest.mark.gpu
@pytest.mark.parametrize("side", ["left", "right"])
def test_swa_padded_batch_forward_and_backward(lo, side):
    """attention_mask: every batch entry attends over its own real tokens only, padding rows come back zero and
    receive no gradient (the reference's unpad -> varlen attention -> pad branch)."""
    import lact_b200
    from oracle import lact_oracle as orc
    b, l, h, d, window = 3, 300, 2, 64, 96
    lens = [300, 1, 170]
    mask = torch.zeros(b, l, dtype=torch.int64)
    for i, n in enumerate(lens):
        if side == "right":
            mask[i, :n] = 1
        else:
            mask[i, l - n:] = 1
    g = torch.Generator().manual_seed(29)
    q, k, v = (torch.randn(b, l, h, d, generator=g).to(BF16) for _ in range(3))
    dO = torch.randn(b, l, h, d, generator=g).to(BF16)
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    ref = torch.zeros(b, l, h, d)
    for i in range(b):
        sel = mask[i].bool()
        ref[i, sel] = orc.sliding_window_attention(*(t[i:i + 1, sel] for t in leaves), window)[0]
    (ref * dO.float()).sum().backward()
    cl = [t.cuda().clone().requires_grad_(True) for t in (q, k, v)]
    o = lo.sliding_window_attention(*cl, window, attention_mask=mask.cuda())
    o.backward(dO.cuda())
    lact_b200.synchronize_and_check()
    got = o.detach().float().cpu()
    assert float(got[mask == 0].abs().max()) == 0.0
    assert (got - ref.detach()).abs().max() / ref.detach().abs().max() <= 1.5e-2
    for name, x, want in zip("qkv", cl, leaves):
        a, b_ = x.grad.float().cpu(), want.grad
        assert float(a[mask == 0].abs().max()) == 0.0, name
        assert orc.rel_max(a, b_) <= 3e-2 and orc.cosine(a, b_) >= 0.9995, (name, orc.rel_max(a, b_), orc.cosine(a, b_))
    with pytest.raises(ValueError):
        lo.sliding_window_attention(*[t.detach() for t in cl], window, attention_mask=mask.cuda(),
                                    cu_seqlens=torch.tensor([0, 900], dtype=torch.int32).cuda())


@pytest.mark.gpu
@pytest.mark.parametrize("d,lq,lk", [(128, 300, 300), (128, 200, 457), (64, 390, 130), (128, 1560, 1750), (64, 64, 1),
                                     (128, 1, 700)])   # (one query over a cache of keys: a decoding step)
def test_block_attention_forward_and_backward(lo, d, lq, lk):
    """Not causal, other key count than query count (the autoregressive-video layer's frame blocks): output and
    gradients against fp32 attention with every key visible."""
    import lact_b200
    from oracle import lact_oracle as orc
    b, h = 2, 2
    g = torch.Generator().manual_seed(31)
    q = torch.randn(b, lq, h, d, generator=g).to(BF16)
    k, v = (torch.randn(b, lk, h, d, generator=g).to(BF16) for _ in range(2))
    dO = torch.randn(b, lq, h, d, generator=g).to(BF16)
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    ref = orc.masked_attention(*leaves, torch.ones(lq, lk, dtype=torch.bool))
    (ref * dO.float()).sum().backward()
    cl = [t.cuda().clone().requires_grad_(True) for t in (q, k, v)]
    o = lo.block_attention(*cl)
    o.backward(dO.cuda())
    lact_b200.synchronize_and_check()
    assert (o.detach().float().cpu() - ref.detach()).abs().max() / ref.detach().abs().max() <= 1.5e-2
    for name, x, want in zip("qkv", cl, leaves):
        a, b_ = x.grad.float().cpu(), want.grad
        assert a.shape == b_.shape
        if float(b_.abs().max()) == 0.0:   # one key: the probabilities are constant, dq and dk vanish
            assert float(a.abs().max()) <= 1e-2, name
        else:
            assert orc.rel_max(a, b_) <= 3e-2 and orc.cosine(a, b_) >= 0.9995, (name, orc.rel_max(a, b_), orc.cosine(a, b_))


@pytest.mark.gpu
@pytest.mark.parametrize("repeated", [False, True])
def test_ar_video_block_attention_matches_the_visibility_matrix(lo, repeated):
    """batched_sliding_window_attention[_with_repeated_chunks]: the reshaped block calls against ONE masked attention
    over the whole sequence with the visibility matrix restated from the reference's structure; forward and backward."""
    import lact_b200
    from oracle import lact_oracle as orc
    mb, kvc, num_chunks = 150, 70, 3
    ue = 3 * mb if repeated else 2 * mb
    l = ue - mb + ue * (num_chunks - 1)
    b, h, d = 2, 2, 128
    g = torch.Generator().manual_seed(37)
    q, k, v = (torch.randn(b, l, h, d, generator=g).to(BF16) for _ in range(3))
    dO = torch.randn(b, l, h, d, generator=g).to(BF16)
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    ref = orc.masked_attention(*leaves, orc.ar_block_visibility(l, mb, ue, num_chunks, kvc, repeated))
    (ref * dO.float()).sum().backward()
    cl = [t.cuda().clone().requires_grad_(True) for t in (q, k, v)]
    fn = lo.batched_sliding_window_attention_with_repeated_chunks if repeated else lo.batched_sliding_window_attention
    o = fn(*cl, mb, ue, num_chunks, kvc)
    o.backward(dO.cuda())
    lact_b200.synchronize_and_check()
    assert o.shape == q.shape
    assert (o.detach().float().cpu() - ref.detach()).abs().max() / ref.detach().abs().max() <= 1.5e-2
    for name, x, want in zip("qkv", cl, leaves):
        a, b_ = x.grad.float().cpu(), want.grad
        assert orc.rel_max(a, b_) <= 3e-2 and orc.cosine(a, b_) >= 0.9995, (name, orc.rel_max(a, b_), orc.cosine(a, b_))


@pytest.mark.gpu
def test_ar_video_inference_attention_three_cases(lo):
    """sliding_window_attention_inference: plain, interleaved (clean + noisy part) and with a key / value cache."""
    import lact_b200
    from oracle import lact_oracle as orc
    b, h, d, mb, kvc = 2, 2, 128, 140, 60
    g = torch.Generator().manual_seed(41)
    q, k, v = (torch.randn(b, 2 * mb, h, d, generator=g).to(BF16) for _ in range(3))
    cache = torch.randn(2 * b, kvc, h, d, generator=g).to(BF16)
    cu = lambda *ts: [t.cuda() for t in ts]
    close = lambda got, ref: float((got.float().cpu() - ref).abs().max() / ref.abs().max()) <= 1.5e-2
    # (1) plain
    got = lo.sliding_window_attention_inference(*cu(q, k, v), mb)
    assert close(got, orc.masked_attention(q, k, v, torch.ones(2 * mb, 2 * mb, dtype=torch.bool)))
    # (2) interleaved: clean block, then the noisy block over the last kvc clean keys and itself
    vis = torch.zeros(2 * mb, 2 * mb, dtype=torch.bool)
    vis[:mb, :mb] = True
    vis[mb:, mb - kvc:] = True
    got = lo.sliding_window_attention_inference(*cu(q, k, v), mb, interleave=True, kv_cache_size=kvc)
    assert close(got, orc.masked_attention(q, k, v, vis))
    # (3) cache of all entries' keys, then values
    got = lo.sliding_window_attention_inference(*cu(q, k, v), mb, kv_cache=cache.cuda())
    kc, vc = cache[:b], cache[b:]
    ref = orc.masked_attention(q, torch.cat([kc, k], 1), torch.cat([vc, v], 1), torch.ones(2 * mb, kvc + 2 * mb, dtype=torch.bool))
    assert close(got, ref)
    lact_b200.synchronize_and_check()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["window", "causal", "block", "packed"])
def test_swa_against_the_flash_attn_library_when_installed(lo, mode):
    """The calls the reference layer makes (flash_attn_func / flash_attn_varlen_func, flash-attn as installed on the
    test machine) on the same bf16 inputs: outputs and gradients of the two bf16 implementations agree to bf16
    accuracy.  Skipped where the library is not importable."""
    fa = pytest.importorskip("flash_attn")
    import lact_b200
    b, l, h, d, w = 2, 3000, 4, 128, 700
    g = torch.Generator().manual_seed(43)
    q, k, v = (torch.randn(b, l, h, d, generator=g).to(BF16).cuda() for _ in range(3))
    dO = torch.randn(b, l, h, d, generator=g).to(BF16).cuda()
    cu = torch.tensor([0, 500, 1777, 3000], dtype=torch.int32).cuda()
    if mode == "packed":
        q, k, v, dO = (t[:1].contiguous() for t in (q, k, v, dO))
    mine = [t.clone().requires_grad_(True) for t in (q, k, v)]
    ref = [t.clone().requires_grad_(True) for t in (q, k, v)]
    if mode == "window":
        o = lo.sliding_window_attention(*mine, w)
        o_ref = fa.flash_attn_func(*ref, causal=True, window_size=(w - 1, 0))
    elif mode == "causal":
        o = lo.sliding_window_attention(*mine, None)
        o_ref = fa.flash_attn_func(*ref, causal=True)
    elif mode == "block":
        o = lo.block_attention(*mine)
        o_ref = fa.flash_attn_func(*ref, causal=False)
    else:
        o = lo.sliding_window_attention(*mine, w, cu_seqlens=cu)
        o_ref = fa.flash_attn_varlen_func(*(t[0] for t in ref), cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=1277,
                                          max_seqlen_k=1277, causal=True, window_size=(w - 1, 0)).unsqueeze(0)
    o.backward(dO)
    o_ref.backward(dO)
    lact_b200.synchronize_and_check()
    rel = lambda a, b_: float((a.float() - b_.float()).abs().max() / b_.float().abs().max())
    cos = lambda a, b_: float(torch.nn.functional.cosine_similarity(a.float().flatten(), b_.float().flatten(), dim=0))
    assert rel(o.detach(), o_ref.detach()) <= 1.5e-2, rel(o.detach(), o_ref.detach())
    for name, a, b_ in zip("qkv", mine, ref):
        assert rel(a.grad, b_.grad) <= 3e-2 and cos(a.grad, b_.grad) >= 0.9995, (name, rel(a.grad, b_.grad), cos(a.grad, b_.grad))
