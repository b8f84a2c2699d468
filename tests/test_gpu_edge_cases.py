"""Edge cases of the chunk drivers on the GPU: sequences shorter than a chunk, ragged tails, head
dimensions that are not multiples of the tile sizes, strided activation views, the benchmark
configurations' head shapes at reduced length (D = H = 192; D = 128, H = 256; 1560-token frames)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
ARGS = ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")


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


def _inputs(orc, B, L, D, H, seed):
    i = orc.make_inputs(B, L, D, H, seed=seed)
    for n in ("q", "k", "v"):
        i[n] = i[n].to(BF16)
    return i


def _close(orc, got, ref, tol=2e-2, cos=0.999, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape
    assert torch.isfinite(got).all(), what
    assert orc.rel_max(got, ref) <= tol and orc.cosine(got, ref) >= cos, (what, orc.rel_max(got, ref), orc.cosine(got, ref))


@pytest.mark.parametrize("L,C", [(50, 64), (64, 64), (65, 64), (1, 16), (130, 33), (257, 256)])
def test_short_and_ragged_sequences(lb, orc, L, C):
    i = _inputs(orc, 2, L, 64, 64, seed=31)
    ref = orc.block_causal_lact_swiglu_fused(*[i[n] for n in ARGS], chunk_size=C, use_muon=False,
                                             momentum=i["momentum"])
    o = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(*[i[n].cuda() for n in ARGS], chunk_size=C,
                                                                 use_muon=False, momentum=i["momentum"].cuda())
    assert o.shape == (2, L, 64)
    _close(orc, o, ref, what=f"L={L} C={C}")
    lb.synchronize_and_check()


@pytest.mark.parametrize("D,H", [(192, 192), (128, 256), (64, 80), (80, 64), (48, 176), (512, 512)])
def test_head_shapes(lb, orc, D, H):
    """Tile-unaligned and benchmark head shapes, Muon on for the first update only being compared."""
    i = _inputs(orc, 2, 384, D, H, seed=32)
    ref = orc.block_causal_lact_swiglu_fused(*[i[n] for n in ARGS], chunk_size=128, use_muon=False,
                                             momentum=i["momentum"])
    c = {n: i[n].cuda() for n in i}
    o = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(*[c[n] for n in ARGS], chunk_size=128,
                                                                 use_muon=False, momentum=c["momentum"])
    _close(orc, o, ref, what=f"D={D} H={H} muon off")
    refm = orc.block_causal_lact_swiglu_fused(*[i[n] for n in ARGS], chunk_size=128, use_muon=True,
                                              momentum=i["momentum"])
    om = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(*[c[n] for n in ARGS], chunk_size=128,
                                                                  use_muon=True, momentum=c["momentum"])
    _close(orc, om[:, :128], refm[:, :128], what=f"D={D} H={H} muon chunk 0")
    assert orc.cosine(om[:, 128:256].float().cpu(), refm[:, 128:256].float()) >= 0.995
    assert torch.isfinite(om.float()).all()
    lb.synchronize_and_check()


def test_strided_activation_views(lb, orc):
    """q, k, v given as views into one fused [b, l, 3d] projection output (token stride 3d)."""
    i = _inputs(orc, 2, 300, 64, 128, seed=33)
    fused = torch.cat([i["q"], i["k"], i["v"]], dim=-1).cuda()
    q, k, v = fused[..., :64], fused[..., 64:128], fused[..., 128:]
    assert not q.is_contiguous()
    c = {n: i[n].cuda() for n in i}
    o_view = lb.block_causal_lact_swiglu(c["w0"], c["w1"], c["w2"], q, k, v, c["lr0"], c["lr1"], c["lr2"],
                                         chunk_size=100, use_muon=True, momentum=c["momentum"])
    o_cont = lb.block_causal_lact_swiglu(*[c[n] for n in ARGS], chunk_size=100, use_muon=True,
                                         momentum=c["momentum"])
    assert torch.equal(o_view, o_cont)


def test_video_frame_chunks(lb, orc):
    """Config-5 head shape (D = 128, H = 256) with 1560-token frames (not a multiple of any tile)."""
    F_, n_frames = 1560, 3
    i = _inputs(orc, 2, F_ * n_frames, 128, 256, seed=34)
    kw = dict(w_scale=1.0, mini_batch_size=F_, update_every=F_, use_moun=False, weight_norm=True)
    ref = orc.ar_mini_batch(*[i[n].float() for n in ARGS], fw_momentum=i["momentum"], use_momentum=True, **kw)
    c = {n: i[n].cuda() for n in i}
    got = lb.ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum(
        *[c[n] for n in ARGS], fw_momentum=c["momentum"], use_momentum=True, **kw)
    for g, r, nm in zip(got, ref, ("o", "w0", "w1", "w2")):
        _close(orc, g, r, what="video " + nm)


def test_nvs_block_shape(lb, orc):
    """Config-4 structure at reduced size: one update over the input tokens, apply to the targets only."""
    n_in, n_tgt = 3072, 512
    i = _inputs(orc, 2, n_in + n_tgt, 192, 192, seed=35)
    t = lambda w: w.transpose(1, 2).contiguous()
    order = [(0, n_in, True, False), (n_in, n_in + n_tgt, False, True)]
    f = {n: i[n].float() for n in i}
    ref = orc.nvs_mini_batch_apply(t(f["w0"]), t(f["w1"]), t(f["w2"]), f["q"], f["k"], f["v"], f["lr0"], f["lr1"],
                                   f["lr2"], order, muon_update_steps=0)
    c = {n: i[n].cuda() for n in i}
    got = lb.fast_weight_swish_glu_weight_norm_mini_batch_apply(
        t(c["w0"]), t(c["w1"]), t(c["w2"]), c["q"], c["k"], c["v"], c["lr0"], c["lr1"], c["lr2"],
        [lb.TTTOperator(*op) for op in order], muon_update_steps=0)
    assert got[0].shape == (2, n_tgt, 192)
    for g, r, nm in zip(got, ref, ("o", "w0", "w1", "w2")):
        _close(orc, g, r, tol=2e-2, what="nvs " + nm)


def test_host_pipeline_matches_direct_call(lb):
    """Pinned host tensors streamed through the device in slabs of (batch x head) entries give the
    bits of one call on device tensors (entries are independent recurrences)."""
    from lact_b200.host_io import HostPipeline
    from oracle import lact_oracle as orc
    i = orc.make_inputs(8, 600, 64, 64, seed=31, act_dtype=torch.bfloat16)
    names = ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")
    fn = lambda **kw: lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        *[kw[n] for n in names], chunk_size=128, use_muon=True, momentum=kw["momentum"])
    direct = fn(**{k: v.cuda() for k, v in i.items() if torch.is_tensor(v)})
    host = {k: v.pin_memory() for k, v in i.items() if torch.is_tensor(v)}
    out = torch.empty(direct.shape, dtype=direct.dtype).pin_memory()
    pipe = HostPipeline(fn, host, out, n_slabs=4, device=torch.device("cuda", 0))
    for _ in range(2):
        out.zero_()
        pipe.run()
        torch.cuda.synchronize()
        assert torch.equal(out, direct.cpu())
    with pytest.raises(ValueError):
        HostPipeline(fn, host, out, n_slabs=3, device=torch.device("cuda", 0))
    lb.synchronize_and_check()
