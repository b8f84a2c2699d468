"""Index arithmetic of the chunk drivers: the product's step programs against the traces the
CPU oracle records while executing the reference's loops (integer work: bit-exact)."""
import itertools

import pytest
import torch

from lact_b200 import program as P
from oracle import lact_oracle as orc

KIND = {"apply": P.APPLY, "update": P.UPDATE}


def _norm(trace):
    # the oracle records empty apply ranges too; drop them on both sides
    return [(KIND[k], s, e, o) if k == "apply" else (KIND[k], s, e, 0) for k, s, e, o in trace if e > s]


def _drop_empty(steps):
    return [s for s in steps if s[2] > s[1]]


def _tiny(B, L, D=16, H=16):
    return orc.make_inputs(B, L, D, H, seed=0)


@pytest.mark.parametrize("L,C", [(64, 16), (65, 16), (63, 16), (16, 16), (10, 16), (17, 16), (1, 1), (100, 7),
                                 (128, 128), (129, 128), (4096, 2048)])
def test_causal_program(L, C):
    i = _tiny(1, L)
    tr = []
    orc.block_causal_lact_swiglu(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"], i["lr2"],
                                 chunk_size=C, trace=tr)
    assert _drop_empty(P.causal_program(L, C)) == _norm(tr)
    tr2 = []
    orc.block_causal_lact_swiglu_fused(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"],
                                       i["lr2"], chunk_size=C, trace=tr2)
    assert _drop_empty(P.causal_program(L, C)) == _norm(tr2)


def test_bidirectional_program():
    i = _tiny(1, 40)
    tr = []
    orc.bidirectional_lact_swiglu(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"], i["lr2"],
                                  use_muon=False, trace=tr)
    assert P.bidirectional_program(40) == _norm(tr)


@pytest.mark.parametrize("order", [
    [(0, 48, True, False), (0, 64, False, True)],
    [(0, 32, True, True), (32, 64, True, False), (40, 64, False, True)],
    [(0, 64, True, True)],
    [(0, 16, False, True), (0, 16, True, False), (0, 16, False, True), (16, 100, False, True)],
])
def test_operator_list_program(order):
    L = 64
    i = _tiny(1, L)
    t = lambda w: w.transpose(1, 2).contiguous()
    tr = []
    o, *_ = orc.nvs_mini_batch_apply(t(i["w0"]), t(i["w1"]), t(i["w2"]), i["q"], i["k"], i["v"], i["lr0"], i["lr1"],
                                     i["lr2"], order, muon_update_steps=0, trace=tr)
    steps, out_len = P.operator_list_program(order, L)
    assert _drop_empty(steps) == _norm(tr)
    assert out_len == o.shape[1]


@pytest.mark.parametrize("L,mini,every,ulen,rep", [
    (448, 64, 128, -1, 1), (320, 80, 80, -1, 2), (256, 64, 64, -1, 1), (300, 64, 128, -1, 1), (256, -1, -1, -1, 1),
    (390, 78, 78, -1, 1), (512, 64, 192, 400, 1), (100, 30, 45, -1, 3)])
def test_ar_train_program(L, mini, every, ulen, rep):
    i = _tiny(1, L)
    tr = []
    orc.ar_mini_batch(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"], i["lr2"], 1.0,
                      num_repeat=rep, mini_batch_size=mini, update_length=ulen, update_every=every, trace=tr)
    assert _drop_empty(P.ar_train_program(L, mini, ulen, every, rep)) == _norm(tr)


@pytest.mark.parametrize("L,mini,upd,rep", [(200, 120, True, 1), (200, -1, True, 2), (200, 120, False, 1),
                                             (64, 500, True, 1)])
def test_ar_inference_program(L, mini, upd, rep):
    i = _tiny(1, L)
    tr = []
    orc.ar_mini_batch_inference(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"], i["lr2"], 1.0,
                                num_repeat=rep, mini_batch_size=mini, do_update=upd, trace=tr)
    assert P.ar_inference_program(L, mini, upd, rep) == _norm(tr)


def test_bad_chunk_size():
    with pytest.raises(ValueError):
        P.causal_program(10, 0)


def test_registered_operator_shapes_under_fake_tensors():
    """The recurrence is a registered operator (`lact_b200::scan_fwd`) with a shape-only
    implementation, so a tracing compiler sees one opaque node: under FakeTensorMode the public
    functions return tensors of the reference's shapes and dtypes without touching the library."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode
    import lact_b200
    with FakeTensorMode():
        B, L, D, H = 2, 520, 64, 128
        w0 = torch.empty(B, H, D, device="cuda")
        w1 = torch.empty(B, D, H, device="cuda")
        q = torch.empty(B, L, D, device="cuda", dtype=torch.bfloat16)
        lr = torch.empty(B, L, 1, device="cuda")
        o = lact_b200.postnorm_block_causal_lact_swiglu_fused_kernel_triton(w0, w1, w0, q, q, q, lr, lr, lr, chunk_size=128,
                                                                            use_muon=True, momentum=lr)
        assert o.shape == (B, L, D) and o.dtype == torch.bfloat16
        res = lact_b200.ar_fast_weight_swish_glu_weight_norm_mini_batch_inference_with_momentum(
            w0, w1, w0, q, q, q, lr, lr, lr, 1.0, mini_batch_size=260, do_update=True, use_moun=True, num_moun_iters=5,
            fw_momentum=lr, use_momentum=True)
        assert len(res) == 7 and res[1].shape == (B, H, D) and res[5].shape == (B, D, H) and res[4].dtype == torch.float32
        t = lambda w: w.transpose(1, 2)
        o2, a, b, c = lact_b200.fast_weight_swish_glu_weight_norm_mini_batch_apply(
            t(w0), t(w1), t(w0), q, q, q, lr, lr, lr, [lact_b200.TTTOperator(0, 400, True, False),
                                                         lact_b200.TTTOperator(400, 520, False, True)], muon_update_steps=5)
        assert o2.shape == (B, 120, D) and a.shape == (B, D, H) and b.shape == (B, H, D)
        o3 = lact_b200.bidirectional_lact_swiglu(w0, w1, w0, q.float(), q.float(), q.float(), lr, lr, lr)
        assert o3.dtype == torch.float32
