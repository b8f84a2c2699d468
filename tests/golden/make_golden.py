"""Generates tests/golden/ref_outputs.pt by RUNNING THE REFERENCE's own functions on CPU.

Run where the reference tree is available (LACT_REFERENCE_ROOT, default: a `reference` directory beside this
repository):

    python tests/golden/make_golden.py              # chunk drivers and sub-ops -> ref_outputs.pt
    python tests/golden/make_golden.py --prologue   # layer prologue             -> layer_prologue.pt
    python tests/golden/make_golden.py --baseline-shapes   # drivers at the benchmark configurations' head shapes
                                                           # and chunk sizes (token-subsampled) -> baseline_shapes.pt

The reference ships no golden vectors for this path, so these fixtures are outputs of the
reference itself (eager mode, CPU) on seeded inputs produced by `oracle.lact_oracle.make_inputs`.
Inputs are not stored; their float64 checksums are, so generator drift is detected.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_loader  # noqa: E402  (sets TORCHDYNAMO_DISABLE before torch is used)
import torch  # noqa: E402
from oracle import lact_oracle as orc  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_outputs.pt")
BF16 = torch.bfloat16


def checksum(inp: dict) -> float:
    return float(sum(t.double().sum() for t in inp.values()))


def cases():
    """(name, kind, input spec, kwargs).  Shapes are small; D and H are multiples of 64."""
    out = []
    for muon in (False, True):
        for mom in (False, True):
            out.append((f"llm_post_fp32_muon{int(muon)}_mom{int(mom)}", "llm_post",
                        dict(B=1, L=209, D=64, H=64, seed=1), dict(chunk_size=64, use_muon=muon, mom=mom)))
    out.append(("llm_pre_fp32_muon0_mom1", "llm_pre", dict(B=1, L=209, D=64, H=64, seed=2),
                dict(chunk_size=64, use_muon=False, mom=True)))
    out.append(("llm_pre_fp32_muon1_mom1", "llm_pre", dict(B=1, L=192, D=64, H=128, seed=3),
                dict(chunk_size=64, use_muon=True, mom=True)))
    out.append(("llm_post_fp32_short", "llm_post", dict(B=2, L=50, D=64, H=64, seed=4),
                dict(chunk_size=64, use_muon=True, mom=True)))
    out.append(("llm_post_fp32_rect", "llm_post", dict(B=1, L=150, D=128, H=64, seed=5),
                dict(chunk_size=50, use_muon=True, mom=False)))
    for muon in (False, True):
        out.append((f"llm_post_bf16_muon{int(muon)}_mom1", "llm_post_autocast",
                    dict(B=2, L=320, D=64, H=64, seed=6), dict(chunk_size=64, use_muon=muon, mom=True)))
        out.append((f"bidi_fp32_muon{int(muon)}", "bidi", dict(B=2, L=128, D=64, H=64, seed=7),
                    dict(use_muon=muon)))
    for steps in (0, 5):
        out.append((f"nvs_fp32_steps{steps}", "nvs", dict(B=1, L=320, D=64, H=128, seed=8),
                    dict(order=[(0, 192, True, False), (0, 320, False, True)], steps=steps)))
    out.append(("nvs_fp32_multi", "nvs", dict(B=1, L=320, D=64, H=64, seed=9),
                dict(order=[(0, 128, True, True), (128, 256, True, False), (200, 320, False, True)], steps=3)))
    out.append(("ar_train_plain", "ar", dict(B=1, L=448, D=64, H=128, seed=10),
                dict(w_scale=1.0, mini_batch_size=64, update_every=128, use_moun=False)))
    out.append(("ar_train_muon5", "ar", dict(B=1, L=448, D=64, H=128, seed=10),
                dict(w_scale=0.5, mini_batch_size=64, update_every=128, use_moun=True, num_moun_iters=5)))
    out.append(("ar_train_repeat2", "ar", dict(B=1, L=320, D=64, H=64, seed=11),
                dict(w_scale=1.0, num_repeat=2, mini_batch_size=80, update_every=80, use_moun=True,
                     num_moun_iters=3, weight_norm=True)))
    out.append(("ar_train_nonorm", "ar", dict(B=1, L=256, D=64, H=64, seed=12),
                dict(w_scale=1.0, mini_batch_size=64, update_every=64, use_moun=False, weight_norm=False)))
    out.append(("ar_train_momentum", "ar_mom", dict(B=1, L=390, D=64, H=128, seed=13),
                dict(w_scale=1.0, mini_batch_size=78, update_every=78, use_moun=True, num_moun_iters=5,
                     use_momentum=True)))
    out.append(("ar_infer_update", "ar_inf", dict(B=1, L=200, D=64, H=128, seed=14),
                dict(w_scale=1.0, mini_batch_size=120, do_update=True, use_moun=True, num_moun_iters=5)))
    out.append(("ar_infer_noupdate", "ar_inf", dict(B=1, L=200, D=64, H=128, seed=14),
                dict(w_scale=1.0, do_update=False)))
    out.append(("ar_infer_momentum", "ar_inf_mom", dict(B=1, L=200, D=64, H=128, seed=15),
                dict(w_scale=1.0, mini_batch_size=120, do_update=True, use_moun=True, num_moun_iters=5,
                     use_momentum=True)))
    return out


def run_reference(kind: str, inp: dict, kw: dict):
    w0, w1, w2, q, k, v = (inp[n] for n in ("w0", "w1", "w2", "q", "k", "v"))
    lr0, lr1, lr2, beta = inp["lr0"], inp["lr1"], inp["lr2"], inp["momentum"]
    if kind in ("llm_post", "llm_pre", "llm_post_autocast"):
        mod = ref_loader.llm_unfused()
        fn = mod.prenorm_block_causal_lact_swiglu if kind == "llm_pre" else mod.block_causal_lact_swiglu
        mom = beta if kw["mom"] else None
        if kind == "llm_post_autocast":
            with torch.autocast("cpu", dtype=BF16):
                o = fn(w0, w1, w2, q.to(BF16), k.to(BF16), v.to(BF16), lr0, lr1, lr2,
                       chunk_size=kw["chunk_size"], use_muon=kw["use_muon"], momentum=mom)
        else:
            o = fn(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size=kw["chunk_size"], use_muon=kw["use_muon"],
                   momentum=mom)
        return dict(o=o)
    if kind == "bidi":
        return dict(o=ref_loader.bidirectional().bidirectional_lact_swiglu(
            w0, w1, w2, q, k, v, lr0, lr1, lr2, use_muon=kw["use_muon"]))
    if kind == "nvs":
        mod = ref_loader.nvs()
        order = [mod.TTTOperator(*t) for t in kw["order"]]
        t = lambda w: w.transpose(1, 2).contiguous()
        o, a, b, c = mod.fast_weight_swish_glu_weight_norm_mini_batch_apply(
            t(w0), t(w1), t(w2), q, k, v, lr0, lr1, lr2, order, muon_update_steps=kw["steps"])
        return dict(o=o, w0=a, w1=b, w2=c)
    ar = ref_loader.ar_ops()
    if kind == "ar":
        o, a, b, c = ar["ar_fast_weight_swish_glu_weight_norm_mini_batch"](w0, w1, w2, q, k, v, lr0, lr1, lr2, **kw)
        return dict(o=o, w0=a, w1=b, w2=c)
    if kind == "ar_mom":
        o, a, b, c = ar["ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum"](
            w0, w1, w2, q, k, v, lr0, lr1, lr2, fw_momentum=beta, **kw)
        return dict(o=o, w0=a, w1=b, w2=c)
    if kind == "ar_inf":
        o, a, b, c = ar["ar_fast_weight_swish_glu_weight_norm_mini_batch_inference"](
            w0, w1, w2, q, k, v, lr0, lr1, lr2, **kw)
        return dict(o=o, w0=a, w1=b, w2=c)
    if kind == "ar_inf_mom":
        r = ar["ar_fast_weight_swish_glu_weight_norm_mini_batch_inference_with_momentum"](
            w0, w1, w2, q, k, v, lr0, lr1, lr2, fw_momentum=beta, **kw)
        return dict(zip(("o", "w0", "w1", "w2", "m0", "m1", "m2"), r))
    raise KeyError(kind)


def subop_cases():
    """Outputs of the reference's in-file PyTorch reference functions for the fused sub-ops."""
    fh = ref_loader.fused_helpers()
    g = torch.Generator().manual_seed(100)
    B, H, D, L = 2, 128, 64, 200
    W02 = torch.randn(B, 2 * H, D, generator=g) / D ** 0.5
    W1 = torch.randn(B, D, H, generator=g) / H ** 0.5
    X = torch.randn(B, L, D, generator=g)
    V = torch.randn(B, L, D, generator=g)
    l0, l1, l2 = torch.rand(3, B, L, generator=g).unbind(0)
    res = {}
    res["swiglu_ffn_fwd"] = dict(o=fh["reference_swiglu_ffn_fwd"](W02, W1, X))
    a, b = fh["reference_lact_swiglu_ffn_fast_weight_grads"](W02, W1, X, V, l0, l1, l2)
    res["fw_grads"] = dict(dw0w2=a, dw1=b)
    xa = torch.randn(B, 2 * H, D, generator=g) * 0.1
    sc = torch.rand(B, 2 * H, generator=g) + 0.5
    res["l2_norm_add"] = dict(y=fh["reference_l2_norm_add_fused"](W02, xa, sc))
    m = torch.randn(B, 2 * H, D, generator=g) * 0.1
    mu = torch.rand(B, generator=g)
    x_new, m_new, y = fh["reference_l2_norm_add_fused_with_momentum"](W02, xa, m, mu, sc)
    res["prenorm_momentum"] = dict(x=x_new, m=m_new, y=y)
    # Newton-Schulz, both coefficient schedules, square / wide / tall
    llm = ref_loader.llm_unfused()
    nvs = ref_loader.nvs()
    for name, shape in (("sq", (2, 64, 64)), ("wide", (2, 64, 128)), ("tall", (2, 128, 64))):
        G = torch.randn(*shape, generator=g)
        res[f"ns_tuned_{name}"] = dict(x=llm.zeropower_via_newtonschulz5(G))
        for steps in (0, 3, 5):
            res[f"ns_const{steps}_{name}"] = dict(x=nvs.zeropower_via_newtonschulz5(G, steps))
    res["_subop_seed"] = 100
    return res


PROLOGUE_OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "layer_prologue.pt")


def fla_version():
    import fla
    return fla.__version__


def prologue_cases():
    """Fast-weight input prologue of the LLM layer (lact_llm/lact_model/layer_lact_swiglu.py:399-414, the
    `ttt_nope` branch): head split, SiLU on q, k (and v), per-head `l2_norm` of q, k -- executed with the
    reference's own `l2_norm` (ttt_operation.py:19-26), `F.silu` and the same einops patterns, bf16 as under
    the layer's autocast."""
    import torch.nn.functional as F
    from einops import rearrange
    l2_norm = ref_loader.llm_unfused().l2_norm
    res = {}
    for name, (b, s, n_h, d, v_silu, seed) in dict(a=(2, 37, 4, 64, True, 200), b=(1, 130, 2, 384, False, 201),
                                                    c=(3, 16, 3, 192, True, 202)).items():
        g = torch.Generator().manual_seed(seed)
        xq, xk, xv = (torch.randn(b, s, n_h * d, generator=g).to(BF16) * 1.5 for _ in range(3))
        fq, fk, fv = (rearrange(t, "b s (n_h d) -> (b n_h) s d", n_h=n_h) for t in (xq, xk, xv))
        fq, fk = F.silu(fq), F.silu(fk)
        if v_silu:
            fv = F.silu(fv)
        fq, fk = l2_norm(fq), l2_norm(fk)
        res[name] = dict(spec=dict(b=b, s=s, n_h=n_h, d=d, v_silu=v_silu, seed=seed),
                         q=fq.contiguous(), k=fk.contiguous(), v=fv.contiguous())
        print("prologue", name, tuple(fq.shape), fq.dtype)
    # rotary embedding of fast q, k (layer_lact_swiglu.py:417-446): the layer's own module fla.modules.RotaryEmbedding
    # supplies the cos / sin tables (`_update_cos_sin_cache`, pure PyTorch); its rotation kernel is Triton-only, so
    # fla's PyTorch restatement `rotary_embedding_ref` of the same file is executed on the reference's l2-normed q, k
    from fla.modules import RotaryEmbedding
    from fla.modules.rotary import rotary_embedding_ref
    for name, (b, s, n_h, d, hd, off, seed) in dict(rope_a=(2, 37, 4, 64, 64, 0, 230), rope_b=(1, 130, 2, 384, 128, 5, 231),
                                                     rope_c=(2, 16, 2, 128, 32, 3, 232)).items():
        g = torch.Generator().manual_seed(seed)
        xq, xk = (torch.randn(b, s, n_h * d, generator=g).to(BF16) * 1.5 for _ in range(2))
        fq, fk = (l2_norm(F.silu(rearrange(t, "b s (n_h d) -> (b n_h) s d", n_h=n_h))) for t in (xq, xk))
        rot = RotaryEmbedding(dim=hd, base=500000.0)
        rot._update_cos_sin_cache(off + s, device=xq.device, dtype=BF16)
        cos, sin = rot._cos_cached[off:off + s], rot._sin_cached[off:off + s]
        outs = []
        for t in (fq, fk):
            m = rearrange(t, "(b n_h) s d -> b s (n_h d)", n_h=n_h)
            m = rearrange(m, "b s (a hd) -> b s a hd", hd=hd)
            m = rotary_embedding_ref(m, cos, sin)
            m = rearrange(m, "b s a hd -> b s (a hd)")
            outs.append(rearrange(m, "b s (n_h d) -> (b n_h) s d", n_h=n_h).contiguous())
        res[name] = dict(spec=dict(b=b, s=s, n_h=n_h, d=d, hd=hd, off=off, seed=seed), q=outs[0], k=outs[1],
                         cos=rot._cos_cached.clone(), sin=rot._sin_cached.clone(), fla=fla_version())
        print("rope", name, tuple(outs[0].shape), outs[0].dtype)
    # learning rates and momentum of the same layer (layer_lact_swiglu.py:463-480, 245-249): softplus of the fp32
    # projection plus inv_softplus(base_lr), split per head into three [(b n_h), s, 1] tensors; momentum = Sigmoid
    # (inside momentum_proj, bf16 under autocast) then .float(), head-merged
    import math
    for name, (b, s, n_h, base_lr, seed) in dict(lr_a=(2, 37, 4, 1e-2, 210), lr_b=(3, 16, 3, 1e-3, 211)).items():
        g = torch.Generator().manual_seed(seed)
        proj = (torch.randn(b, s, n_h * 3, generator=g) * 2.0).to(BF16)        # lr_proj output under autocast
        mlogit = (torch.randn(b, s, n_h, generator=g) * 2.0).to(BF16)          # momentum Linear output under autocast
        base_lr_inv = base_lr + math.log(-math.expm1(-base_lr))                # inv_softplus, layer_lact_swiglu.py:44-49
        lr = F.softplus(proj.float() + base_lr_inv)
        fw_lr = rearrange(lr, "b s (n_h lr_dim) -> (b n_h) s lr_dim", n_h=n_h)
        l1, l2, l3 = fw_lr.chunk(3, dim=-1)
        mom = rearrange(torch.sigmoid(mlogit).float(), "b s (n_h d) -> (b n_h) s d", n_h=n_h)
        res[name] = dict(spec=dict(b=b, s=s, n_h=n_h, base_lr=base_lr, seed=seed), lr0=l1.contiguous(), lr1=l2.contiguous(),
                         lr2=l3.contiguous(), momentum=mom.contiguous())
        print("lr prologue", name, tuple(l1.shape), l1.dtype, tuple(mom.shape))
    # output epilogue of the same layer (layer_lact_swiglu.py:556-568): per-head RMSNorm of the recurrence's output
    # (`fla.modules.RMSNorm`, a Triton kernel in the reference; its own PyTorch restatement `rms_norm_ref` with
    # upcast=True is executed here), gate silu(ttt_scale_proj(x)), head merge, residual add to the attention output
    import fla
    from fla.modules.layernorm import rms_norm_ref
    for name, (b, s, n_h, d, seed) in dict(out_a=(2, 37, 4, 64, 220), out_b=(1, 50, 2, 384, 221)).items():
        g = torch.Generator().manual_seed(seed)
        fw_x = (torch.randn(b * n_h, s, d, generator=g) * 2.0).to(BF16)
        weight = 1.0 + 0.1 * torch.randn(d, generator=g)
        sproj = (torch.randn(b, s, n_h * d, generator=g) * 1.5).to(BF16)
        o_attn = torch.randn(b, s, n_h * d, generator=g).to(BF16)
        normed = rms_norm_ref(fw_x, weight, None, eps=1e-5, upcast=True)
        scale = rearrange(F.silu(sproj, inplace=False), "b s (n_h d) -> (b n_h) s d", n_h=n_h)
        normed = normed * scale
        merged = rearrange(normed, "(b n_h) s d -> b s (n_h d)", n_h=n_h)
        res[name] = dict(spec=dict(b=b, s=s, n_h=n_h, d=d, seed=seed), out=(o_attn + merged).contiguous(),
                         fla=fla.__version__)
        print("epilogue", name, tuple(merged.shape), merged.dtype)
    return res


BASELINE_OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline_shapes.pt")


def baseline_shape_cases():
    """(name, kind, input spec, kwargs, token stride of the stored subsample): the reference drivers at the head
    shapes and chunk sizes of the benchmark configurations.  Full outputs would be tens of megabytes, so only every
    `stride`-th output token (all heads, all features) is stored; inputs are regenerated from the seed."""
    out = []
    for muon in (False, True):
        # configuration 1: bidirectional layer, fp32, 4 heads of 192, 4096 tokens, one update then apply
        out.append((f"cfg1_bidi_fp32_muon{int(muon)}", "bidi", dict(B=4, L=4096, D=192, H=192, seed=31),
                    dict(use_muon=muon), 64))
        # configuration 2, one batch element: causal LLM op (unfused signature; the fused one needs Triton),
        # bf16 autocast, 4 heads of 384, chunk 2048, 4 chunks, momentum
        out.append((f"cfg2_llm_bf16_muon{int(muon)}", "llm_post_autocast", dict(B=4, L=8192, D=384, H=384, seed=32),
                    dict(chunk_size=2048, use_muon=muon, mom=True), 128))
        # configuration 5: autoregressive video layer, 12 heads of 128, hidden 256, 21 frames of 1560 tokens, momentum
        out.append((f"cfg5_ar_muon{int(muon)}", "ar_mom", dict(B=12, L=32760, D=128, H=256, seed=35),
                    dict(w_scale=1.0, mini_batch_size=1560, update_every=1560, use_moun=muon, num_moun_iters=5,
                         use_momentum=True), 390))
    # configuration 4, one batch element: NVS operator list, 4 heads of 192, one update on 16384 tokens, apply to 4096
    out.append(("cfg4_nvs_steps5", "nvs", dict(B=4, L=20480, D=192, H=192, seed=34),
                dict(order=[(0, 16384, True, False), (16384, 20480, False, True)], steps=5), 64))
    return out


def baseline_shapes_main():
    import time
    blob = {"cases": {}, "torch": torch.__version__}
    for name, kind, spec, kw, stride in baseline_shape_cases():
        t0 = time.time()
        inp = orc.make_inputs(**spec)
        res = run_reference(kind, inp, kw)
        sub = {"o": res["o"].detach()[:, ::stride].contiguous().clone()}
        for wn in ("w0", "w1", "w2"):  # final fast weights: first 8 rows of every head
            if res.get(wn) is not None:
                sub[wn] = res[wn].detach()[:, :8].contiguous().clone()
        blob["cases"][name] = dict(kind=kind, spec=spec, kw=kw, stride=stride, checksum=checksum(inp), out=sub)
        print(f"{name:28s} {time.time() - t0:6.1f} s  " +
              " ".join(f"{k}:{tuple(v.shape)}:{str(v.dtype)[6:]}" for k, v in sub.items()))
    torch.save(blob, BASELINE_OUT)
    print("wrote", BASELINE_OUT, os.path.getsize(BASELINE_OUT) // 1024, "KiB")


def main():
    if "--baseline-shapes" in sys.argv:
        assert ref_loader.available(), "reference tree not found"
        baseline_shapes_main()
        return
    if "--prologue" in sys.argv:
        assert ref_loader.available(), "reference tree not found"
        torch.set_num_threads(1)
        torch.save(prologue_cases(), PROLOGUE_OUT)
        print("wrote", PROLOGUE_OUT, os.path.getsize(PROLOGUE_OUT) // 1024, "KiB")
        return
    assert ref_loader.available(), "reference tree not found"
    torch.set_num_threads(1)  # fixtures must not depend on the thread count
    blob = {"cases": {}, "subops": subop_cases(), "torch": torch.__version__}
    for name, kind, spec, kw in cases():
        inp = orc.make_inputs(**spec)
        res = run_reference(kind, inp, kw)
        blob["cases"][name] = dict(kind=kind, spec=spec, kw=kw, checksum=checksum(inp),
                                   out={k: v.detach().clone() for k, v in res.items() if v is not None})
        print(f"{name:32s} " + " ".join(f"{k}:{tuple(v.shape)}:{str(v.dtype)[6:]}" for k, v in res.items() if v is not None))
    torch.save(blob, OUT)
    print("wrote", OUT, os.path.getsize(OUT) // 1024, "KiB")


if __name__ == "__main__":
    main()
