"""The CPU oracle against outputs of the reference itself (tests/golden/ref_outputs.pt).

With fp32 inputs the oracle's `ref` policy uses the same PyTorch CPU primitives in the same
order as the reference functions, so the comparison is normally bit-exact.  A different host
ISA may change GEMM summation order; the fallback tolerance covers that (after a Muon step the
recurrence amplifies rounding noise to about 1e-2, so Muon cases get the wider band).
"""
import pytest
import torch

from oracle import lact_oracle as orc

BF16 = torch.bfloat16


from oracle_drivers import run_oracle as _run_oracle  # noqa: E402


def _uses_muon(kw):
    return bool(kw.get("use_muon") or kw.get("use_moun") or kw.get("steps", 0) > 0)


def test_all_cases_present(golden):
    assert len(golden["cases"]) == 23


@pytest.mark.parametrize("name", [
    "llm_post_fp32_muon0_mom0", "llm_post_fp32_muon0_mom1", "llm_post_fp32_muon1_mom0", "llm_post_fp32_muon1_mom1",
    "llm_pre_fp32_muon0_mom1", "llm_pre_fp32_muon1_mom1", "llm_post_fp32_short", "llm_post_fp32_rect",
    "llm_post_bf16_muon0_mom1", "llm_post_bf16_muon1_mom1", "bidi_fp32_muon0", "bidi_fp32_muon1",
    "nvs_fp32_steps0", "nvs_fp32_steps5", "nvs_fp32_multi", "ar_train_plain", "ar_train_muon5",
    "ar_train_repeat2", "ar_train_nonorm", "ar_train_momentum", "ar_infer_update", "ar_infer_noupdate",
    "ar_infer_momentum"])
def test_oracle_matches_reference_output(golden, name):
    torch.set_num_threads(1)
    case = golden["cases"][name]
    inp = orc.make_inputs(**case["spec"])
    chk = float(sum(t.double().sum() for t in inp.values()))
    assert abs(chk - case["checksum"]) <= 1e-6 * max(1.0, abs(chk)), "seeded input generator drifted"
    got = _run_oracle(case["kind"], inp, case["kw"])
    tol = 6e-2 if _uses_muon(case["kw"]) else 2e-5
    if case["kind"] == "llm_post_autocast":
        tol = max(tol, 1e-2)
    for key, ref in case["out"].items():
        g = got[key]
        assert g.shape == ref.shape and g.dtype == ref.dtype, key
        if torch.equal(g, ref):
            continue
        assert orc.rel_fro(g, ref) <= tol, (name, key, orc.rel_fro(g, ref))


def test_subops_match_reference_helpers(golden):
    so = golden["subops"]
    g = torch.Generator().manual_seed(so["_subop_seed"])
    B, H, D, L = 2, 128, 64, 200
    W02 = torch.randn(B, 2 * H, D, generator=g) / D ** 0.5
    W1 = torch.randn(B, D, H, generator=g) / H ** 0.5
    X = torch.randn(B, L, D, generator=g)
    V = torch.randn(B, L, D, generator=g)
    l0, l1, l2 = torch.rand(3, B, L, generator=g).unbind(0)
    # fused-policy helpers evaluated in fp32 reproduce the reference formulas
    o = orc.apply_fused(W02, W1, X)
    assert orc.rel_fro(o, so["swiglu_ffn_fwd"]["o"]) < 1e-5
    dw02, dw1 = orc.grads_fused(W02, W1, X, V, l0, l1, l2)
    assert orc.rel_fro(dw02, so["fw_grads"]["dw0w2"]) < 1e-5
    assert orc.rel_fro(dw1, so["fw_grads"]["dw1"]) < 1e-5
    xa = torch.randn(B, 2 * H, D, generator=g) * 0.1
    sc = torch.rand(B, 2 * H, generator=g) + 0.5
    assert orc.rel_fro(orc.l2_norm_add(W02, xa, sc), so["l2_norm_add"]["y"]) < 1e-6
    m = torch.randn(B, 2 * H, D, generator=g) * 0.1
    mu = torch.rand(B, generator=g)
    x_new, m_new, y = orc.prenorm_update_with_momentum(W02, xa, m, mu, sc)
    assert orc.rel_fro(x_new, so["prenorm_momentum"]["x"]) < 1e-6
    assert orc.rel_fro(m_new, so["prenorm_momentum"]["m"]) < 1e-6
    assert orc.rel_fro(y, so["prenorm_momentum"]["y"]) < 1e-2
    for name, shape in (("sq", (2, 64, 64)), ("wide", (2, 64, 128)), ("tall", (2, 128, 64))):
        G = torch.randn(*shape, generator=g)
        x = orc.newton_schulz(G)
        ref = so[f"ns_tuned_{name}"]["x"]
        assert torch.equal(x, ref) or orc.rel_fro(x, ref) < 3e-2
        for steps in (0, 3, 5):
            x = orc.newton_schulz(G, steps)
            ref = so[f"ns_const{steps}_{name}"]["x"]
            assert torch.equal(x, ref) or orc.rel_fro(x, ref) < 3e-2


def test_scan_model_tracks_reference_without_muon(golden):
    """The kernel-rounding model in fp32 mode equals the unfused reference when Muon is off."""
    case = golden["cases"]["llm_post_fp32_muon0_mom1"]
    inp = orc.make_inputs(**case["spec"])
    trace = []
    orc.block_causal_lact_swiglu(inp["w0"], inp["w1"], inp["w2"], inp["q"], inp["k"], inp["v"], inp["lr0"],
                                 inp["lr1"], inp["lr2"], chunk_size=64, momentum=inp["momentum"], trace=trace)
    cfg = orc.ScanConfig(use_muon=False, renorm="outer", fp32_mode=True)
    o, *_ = orc.scan_model(inp["w0"], inp["w1"], inp["w2"], inp["q"], inp["k"], inp["v"], inp["lr0"], inp["lr1"],
                           inp["lr2"], trace, cfg, momentum=inp["momentum"])
    assert orc.rel_max(o, case["out"]["o"]) < 1e-4


def test_layer_prologue_matches_reference_outputs():
    """`qkv_prologue` (silu, per-head l2 norm, head split) against outputs of the reference's own functions
    (tests/golden/layer_prologue.pt, written by make_golden.py --prologue): bit-exact."""
    import os
    import torch
    from oracle import lact_oracle as orc
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    for name, case in blob.items():
        if name.startswith(("lr_", "out_", "rope_")):
            continue
        sp = case["spec"]
        g = torch.Generator().manual_seed(sp["seed"])
        xq, xk, xv = (torch.randn(sp["b"], sp["s"], sp["n_h"] * sp["d"], generator=g).to(torch.bfloat16) * 1.5
                      for _ in range(3))
        q, k, v = orc.qkv_prologue(xq, xk, xv, sp["n_h"], True, sp["v_silu"])
        assert torch.equal(q, case["q"]) and torch.equal(k, case["k"]) and torch.equal(v, case["v"]), name


def test_rotary_prologue_matches_reference_outputs():
    """`qkv_prologue_rope` against the fixtures written with the layer's own RotaryEmbedding tables and fla's PyTorch
    restatement of its rotation (make_golden.py --prologue): the cos / sin tables and, with the `ref` rounding policy,
    the rotated q and k are bit-exact; the fused (single-rounding) policy stays within one bf16 ulp of them."""
    import os
    import torch
    from oracle import lact_oracle as orc
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    names = [n for n in blob if n.startswith("rope_")]
    assert len(names) == 3
    for name in names:
        case = blob[name]
        sp = case["spec"]
        g = torch.Generator().manual_seed(sp["seed"])
        xq, xk = (torch.randn(sp["b"], sp["s"], sp["n_h"] * sp["d"], generator=g).to(torch.bfloat16) * 1.5
                  for _ in range(2))
        cos, sin = orc.rotary_tables(sp["hd"], sp["off"] + sp["s"])
        assert torch.equal(cos, case["cos"]) and torch.equal(sin, case["sin"]), name
        q, k, _ = orc.qkv_prologue_rope(xq, xk, xk, sp["n_h"], sp["hd"], cos, sin, sp["off"], policy="ref")
        assert torch.equal(q, case["q"]) and torch.equal(k, case["k"]), name
        qf, kf, _ = orc.qkv_prologue_rope(xq, xk, xk, sp["n_h"], sp["hd"], cos, sin, sp["off"], policy="fused")
        for got, ref in ((qf, case["q"]), (kf, case["k"])):
            ulp = torch.maximum(ref.float().abs(), torch.tensor(2.0 ** -126)).log2().floor().exp2() * 2.0 ** -7
            # near a cancellation (x cos ~ partner sin) the two roundings of the eager arithmetic are not small
            # relative to the result; against the scale of the inputs (|x| <= 1 after the l2 norm) they are
            assert float(((got.float() - ref.float()).abs() / torch.maximum(ulp, torch.tensor(2.0 ** -10))).max()) <= 1.0, name


def test_lr_prologue_matches_reference_outputs():
    """`lr_prologue` (softplus learning rates, sigmoid momentum, head split) against the reference expressions'
    outputs in tests/golden/layer_prologue.pt: bit-exact."""
    import os
    import torch
    from oracle import lact_oracle as orc
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    seen = 0
    for name, case in blob.items():
        if not name.startswith("lr_"):
            continue
        sp = case["spec"]
        g = torch.Generator().manual_seed(sp["seed"])
        proj = (torch.randn(sp["b"], sp["s"], sp["n_h"] * 3, generator=g) * 2.0).to(torch.bfloat16)
        mlogit = (torch.randn(sp["b"], sp["s"], sp["n_h"], generator=g) * 2.0).to(torch.bfloat16)
        l0, l1, l2, mom = orc.lr_prologue(proj, sp["n_h"], sp["base_lr"], mlogit)
        assert torch.equal(l0, case["lr0"]) and torch.equal(l1, case["lr1"]) and torch.equal(l2, case["lr2"]), name
        assert torch.equal(mom, case["momentum"]), name
        seen += 1
    assert seen == 2


def test_out_epilogue_matches_reference_outputs():
    """`out_epilogue` (per-head RMSNorm, silu gate, head merge, residual add) against the fixture written with
    flash-linear-attention's own `rms_norm_ref` and the layer's expressions: bit-exact."""
    import os
    import torch
    from oracle import lact_oracle as orc
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    seen = 0
    for name, case in blob.items():
        if not name.startswith("out_"):
            continue
        sp = case["spec"]
        b, s, n_h, d = sp["b"], sp["s"], sp["n_h"], sp["d"]
        g = torch.Generator().manual_seed(sp["seed"])
        fw_x = (torch.randn(b * n_h, s, d, generator=g) * 2.0).to(torch.bfloat16)
        weight = 1.0 + 0.1 * torch.randn(d, generator=g)
        sproj = (torch.randn(b, s, n_h * d, generator=g) * 1.5).to(torch.bfloat16)
        o_attn = torch.randn(b, s, n_h * d, generator=g).to(torch.bfloat16)
        assert torch.equal(orc.out_epilogue(fw_x, weight, n_h, sproj, o_attn), case["out"]), name
        seen += 1
    assert seen == 2


@pytest.mark.parametrize("l,window", [(300, 64), (257, None), (130, 1), (96, 200)])
def test_sliding_window_attention_restatement_against_sdpa(l, window):
    """The oracle's banded attention against PyTorch's own scaled_dot_product_attention with the band as an
    explicit mask (an independent implementation of the same published semantics)."""
    from oracle import lact_oracle as orc
    g = torch.Generator().manual_seed(l)
    q, k, v = (torch.randn(2, l, 3, 32, generator=g) for _ in range(3))
    got = orc.sliding_window_attention(q, k, v, window, block=100)
    i = torch.arange(l).view(-1, 1)
    j = torch.arange(l).view(1, -1)
    w = l if window is None else window
    mask = (j <= i) & (j > i - w)
    ref = torch.nn.functional.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3),
                                                           v.permute(0, 2, 1, 3), attn_mask=mask).permute(0, 2, 1, 3)
    assert torch.allclose(got, ref, atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("repeated", [False, True])
def test_ar_block_visibility_equals_the_block_by_block_calls(repeated):
    """The one-matrix restatement of the autoregressive-video layer's attention against a literal replay of the
    reference's structure (ar_lact_swa_repeat.py:299-463: reshape into blocks, one full attention per block group)
    with PyTorch's scaled_dot_product_attention standing in for the flash-attn call."""
    import torch.nn.functional as F
    from einops import rearrange, repeat
    mb, kvc, num_chunks = 6, 4, 3
    ue = 3 * mb if repeated else 2 * mb
    first = ue - mb
    l = first + ue * (num_chunks - 1)
    b, h, d = 2, 2, 8
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(b, l, h, d, generator=g) for _ in range(3))
    full = lambda q_, k_, v_: F.scaled_dot_product_attention(q_.transpose(1, 2), k_.transpose(1, 2), v_.transpose(1, 2)).transpose(1, 2)
    o = torch.zeros_like(q)
    nr = ue // mb - 1
    if repeated:
        blk = lambda t: rearrange(t[:, :first], "b (nr fw) h d -> (b nr) fw h d", nr=nr)
        o[:, :first] = rearrange(full(blk(q), blk(k), blk(v)), "(b nr) fw h d -> b (nr fw) h d", nr=nr)
    else:
        o[:, :first] = full(q[:, :first], k[:, :first], v[:, :first])
    q_r, k_r, v_r = (rearrange(t[:, first:], "b (n_c sw) h d -> (b n_c) sw h d", sw=ue) for t in (q, k, v))
    o_clean = full(q_r[:, :mb], k_r[:, :mb], v_r[:, :mb])
    if repeated:
        nz = lambda t: rearrange(t[:, mb:], "b (n_repeat sw) h d -> (b n_repeat) sw h d", n_repeat=nr)
        rp = lambda t: repeat(t[:, :mb][:, -kvc:], "b sw h d -> (b n_repeat) sw h d", n_repeat=nr)
        o_noise = full(nz(q_r), torch.cat([rp(k_r), nz(k_r)], 1), torch.cat([rp(v_r), nz(v_r)], 1))
        o_noise = rearrange(o_noise, "(b n_repeat) sw h d -> b (n_repeat sw) h d", n_repeat=nr)
    else:
        o_noise = full(q_r[:, mb:], k_r[:, mb - kvc:], v_r[:, mb - kvc:])
    o[:, first:] = rearrange(torch.cat([o_clean, o_noise], 1), "(b n_c) sw h d -> b (n_c sw) h d", n_c=num_chunks - 1)
    got = orc.masked_attention(q, k, v, orc.ar_block_visibility(l, mb, ue, num_chunks, kvc, repeated))
    assert torch.allclose(got, o, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("l,w", [(37, 5), (64, 64), (50, None)])
def test_banded_attention_equals_masked_attention(l, w):
    """Two restatements of the same semantics: the blocked banded attention and one masked attention with the band
    written out as a visibility matrix (the form the block-attention checks use)."""
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(2, l, 2, 16, generator=g) for _ in range(3))
    i, j = torch.arange(l).view(-1, 1), torch.arange(l).view(1, -1)
    vis = (j <= i) & (j > i - (w if w else l))
    assert torch.allclose(orc.sliding_window_attention(q, k, v, w, block=16), orc.masked_attention(q, k, v, vis),
                          atol=1e-5, rtol=1e-5)


def test_sequence_start_index_of_packed_sequences():
    """The per-token sequence-start array the attention and rotary kernels take, from cu_seqlens (host-side helper)."""
    from lact_b200.layer_ops import _seq_start
    cu = torch.tensor([0, 3, 4, 9], dtype=torch.int32)
    assert _seq_start(cu, 9, "cpu").tolist() == [0, 0, 0, 3, 4, 4, 4, 4, 4]
    assert _seq_start(cu, 9, "cpu").dtype == torch.int32


def test_exported_l2_norm_reproduces_the_reference_outputs():
    """`lact_b200.l2_norm` (the helper the reference layer imports beside the chunk drivers) on SiLU'd, head-split
    projections: bit-exact against the fixture written by the reference's own `l2_norm`."""
    import os
    import torch.nn.functional as F
    import lact_b200
    blob = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_prologue.pt"),
                      map_location="cpu", weights_only=False)
    case = blob["a"]
    sp = case["spec"]
    g = torch.Generator().manual_seed(sp["seed"])
    xq = torch.randn(sp["b"], sp["s"], sp["n_h"] * sp["d"], generator=g).to(torch.bfloat16) * 1.5
    heads = xq.reshape(sp["b"], sp["s"], sp["n_h"], sp["d"]).permute(0, 2, 1, 3).reshape(sp["b"] * sp["n_h"], sp["s"], sp["d"])
    assert torch.equal(lact_b200.l2_norm(F.silu(heads)), case["q"])
