"""Shared by the oracle and GPU tests: runs the CPU oracle's driver that corresponds to a fixture kind
(the kinds are those of tests/golden/make_golden.py)."""
import torch

from oracle import lact_oracle as orc

BF16 = torch.bfloat16


def run_oracle(kind, inp, kw):
    w0, w1, w2, q, k, v = (inp[n] for n in ("w0", "w1", "w2", "q", "k", "v"))
    lr0, lr1, lr2, beta = inp["lr0"], inp["lr1"], inp["lr2"], inp["momentum"]
    if kind in ("llm_post", "llm_pre"):
        o = orc.block_causal_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size=kw["chunk_size"],
                                         use_muon=kw["use_muon"], momentum=beta if kw["mom"] else None,
                                         prenorm=(kind == "llm_pre"))
        return dict(o=o)
    if kind == "llm_post_autocast":
        o = orc.block_causal_lact_swiglu(w0, w1, w2, q.to(BF16), k.to(BF16), v.to(BF16), lr0, lr1, lr2,
                                         chunk_size=kw["chunk_size"], use_muon=kw["use_muon"],
                                         momentum=beta if kw["mom"] else None,
                                         nm=orc.Numerics("ref", autocast=True))
        return dict(o=o)
    if kind == "bidi":
        return dict(o=orc.bidirectional_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, use_muon=kw["use_muon"]))
    if kind == "nvs":
        t = lambda w: w.transpose(1, 2).contiguous()
        o, a, b, c = orc.nvs_mini_batch_apply(t(w0), t(w1), t(w2), q, k, v, lr0, lr1, lr2, kw["order"],
                                              muon_update_steps=kw["steps"])
        return dict(o=o, w0=a, w1=b, w2=c)
    if kind == "ar":
        return dict(zip(("o", "w0", "w1", "w2"), orc.ar_mini_batch(w0, w1, w2, q, k, v, lr0, lr1, lr2, **kw)))
    if kind == "ar_mom":
        return dict(zip(("o", "w0", "w1", "w2"),
                        orc.ar_mini_batch(w0, w1, w2, q, k, v, lr0, lr1, lr2, fw_momentum=beta, **kw)))
    if kind == "ar_inf":
        return dict(zip(("o", "w0", "w1", "w2"),
                        orc.ar_mini_batch_inference(w0, w1, w2, q, k, v, lr0, lr1, lr2, **kw)))
    if kind == "ar_inf_mom":
        return dict(zip(("o", "w0", "w1", "w2", "m0", "m1", "m2"),
                        orc.ar_mini_batch_inference(w0, w1, w2, q, k, v, lr0, lr1, lr2, fw_momentum=beta,
                                                    with_momentum_api=True, **kw)))
    raise KeyError(kind)
