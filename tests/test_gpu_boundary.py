"""Behaviour of the drop-in boundary that is not arithmetic: no host synchronisation on the hot
path, the bounded-wait status path (made to run out WITHOUT any fault: a thread waits on a barrier
nobody arrives on), recovery after a recorded failure, gradients through the returned fast
weights, and zero-filled gaps of the output."""
import ctypes as C

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


@pytest.fixture(scope="module")
def orc():
    from oracle import lact_oracle
    return lact_oracle


def _inputs(orc, B, L, D, H, seed):
    i = orc.make_inputs(B, L, D, H, seed=seed)
    for n in ("q", "k", "v"):
        i[n] = i[n].to(BF16)
    return i


def test_back_to_back_calls_never_synchronise(lb, orc):
    """20 calls of a driver and of a fused sub-op in a row: the library waits for the stream in
    lact_read_status / lact_static_status only, and the Python shim does not call them on the hot path."""
    from lact_b200 import _lib as LL
    i = {k: v.cuda() for k, v in _inputs(orc, 2, 512, 64, 64, seed=1).items()}
    args = [i[n] for n in NAMES]
    lb.block_causal_lact_swiglu(*args, chunk_size=128, use_muon=True, momentum=i["momentum"])  # warm-up
    lb.synchronize_and_check()
    w02 = torch.cat([i["w0"], i["w2"]], dim=1).to(BF16)
    w1 = i["w1"].to(BF16)
    before = LL.stream_sync_count()
    outs = []
    for _ in range(20):
        outs.append(lb.block_causal_lact_swiglu(*args, chunk_size=128, use_muon=True, momentum=i["momentum"]))
        outs.append(lb.fused_swiglu_ffn_fwd(w02, w1, i["q"]))
    assert LL.stream_sync_count() == before, "a library call synchronised the stream"
    lb.synchronize_and_check()
    assert LL.stream_sync_count() == before
    assert all(torch.equal(outs[0], o) for o in outs[2::2])


def test_training_step_never_synchronises(lb, orc):
    """Forward + backward of a driver with PyTorch's synchronisation detector armed: any blocking call on the
    host path (an .item(), a blocking copy, a stream wait) raises."""
    from lact_b200 import _lib as LL
    i = _inputs(orc, 2, 512, 64, 64, seed=6)
    dO = torch.randn(2, 512, 64).to(BF16).cuda()

    def step():
        leaves = {n: i[n].cuda().requires_grad_(True) for n in NAMES}
        mom = i["momentum"].cuda().requires_grad_(True)
        o = lb.block_causal_lact_swiglu(*[leaves[n] for n in NAMES], chunk_size=128, use_muon=True, momentum=mom)
        o.backward(dO)
        return leaves["k"].grad

    g_ref = step()  # warm-up: allocations, pinned ring
    lb.synchronize_and_check()
    i = {k_: v_.cuda() for k_, v_ in i.items()}
    before = LL.stream_sync_count()
    torch.cuda.set_sync_debug_mode("error")
    try:
        g = step()
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert LL.stream_sync_count() == before
    lb.synchronize_and_check()
    assert torch.equal(g, g_ref)


def test_bounded_wait_runs_out_is_reported_and_the_next_call_is_clean(lb, orc):
    """A wait that nothing satisfies gives up after the configured limit and leaves status 101 in the
    workspace; the shim turns it into LactError; the workspace is usable again afterwards."""
    from lact_b200 import _lib as LL
    lib = LL.lib()
    i = {k: v.cuda() for k, v in _inputs(orc, 1, 256, 64, 64, seed=2).items()}
    args = [i[n] for n in NAMES]
    ref = lb.block_causal_lact_swiglu(*args, chunk_size=128)
    lb.synchronize_and_check()
    dev = i["q"].device
    ws = LL.workspace(1 << 20, dev)
    try:
        LL.check(lib.lact_set_wait_limit_ns(1_000_000), "lact_set_wait_limit_ns")  # 1 ms
        ws[:256].zero_()
        LL.check(lib.lact_debug_wait_timeout(ws.data_ptr(), LL.stream_ptr()), "lact_debug_wait_timeout")
        # raw C ABI: the status word reads 101
        assert lib.lact_read_status(ws.data_ptr(), LL.stream_ptr()) == 101
        # shim: the word reaches the host through the non-blocking ring and raises at the next look at it
        with pytest.raises(LL.LactError):
            LL.mark_pending(ws)
            lb.synchronize_and_check()
    finally:
        LL.check(lib.lact_set_wait_limit_ns(0), "lact_set_wait_limit_ns")  # back to the default
    # the same workspace, next call: clean and correct
    again = lb.block_causal_lact_swiglu(*args, chunk_size=128)
    lb.synchronize_and_check()
    assert torch.equal(again, ref)


def test_backward_recovers_after_a_recorded_failure(lb, orc):
    """A non-zero status word left by an earlier backward sweep must not disable the next one."""
    from lact_b200 import backward as bw
    i = _inputs(orc, 1, 256, 64, 64, seed=3)

    def grads():
        leaves = {n: i[n].cuda().clone().requires_grad_(True) for n in NAMES}
        o = lb.block_causal_lact_swiglu(*[leaves[n] for n in NAMES], chunk_size=128)
        o.float().sum().backward()
        return leaves["k"].grad.clone()

    g_ref = grads()
    dev = torch.device("cuda", torch.cuda.current_device())
    bw._status_word(dev)[0] = 101  # as if a bounded wait had run out in an earlier sweep
    with pytest.raises(lb.LactError):
        bw.check_status(dev)
    assert int(bw._status_word(dev)[0].item()) == 0  # cleared by the check that raised
    bw._status_word(dev)[0] = 101
    g = grads()  # the sweep clears the word before it starts
    assert torch.equal(g, g_ref)


def test_gradient_through_returned_fast_weights(lb, orc):
    """The final fast weights returned by the state-carrying drivers are differentiable outputs (in the
    reference they carry autograd history, ar_lact_swa_repeat.py:168): a loss that uses them must send
    its gradient back through the recurrence.  Muon off, against autograd through the CPU oracle."""
    B, L, D, H, mb = 2, 512, 64, 128, 128
    i = _inputs(orc, B, L, D, H, seed=4)
    g = torch.Generator().manual_seed(9)
    dO = torch.randn(B, L, D, generator=g).to(BF16)
    r0, r1, r2 = torch.randn(B, H, D, generator=g), torch.randn(B, D, H, generator=g), torch.randn(B, H, D, generator=g)

    def run(fn, dev):
        # oracle: fp32 arithmetic on the bf16-rounded activations; CUDA: bf16 activations as given
        leaves = {n: (i[n].float() if dev == "cpu" else i[n].to(dev)).clone().requires_grad_(True) for n in NAMES}
        o, a, b, c = fn(*[leaves[n] for n in NAMES], 1.0, mini_batch_size=mb, update_every=mb, use_moun=False)
        loss = (o.float() * dO.to(dev).float()).sum() + 50.0 * ((a * r0.to(dev)).sum() + (b * r1.to(dev)).sum() +
                                                                (c * r2.to(dev)).sum())
        loss.backward()
        return {n: leaves[n].grad.detach().float().cpu() for n in NAMES}, (a.detach(), b.detach(), c.detach())

    g_ref, _ = run(orc.ar_mini_batch, "cpu")
    g_cu, _ = run(lb.ar_fast_weight_swish_glu_weight_norm_mini_batch, "cuda")
    # the weight-only part of the loss: without the cotangent seed these gradients would lack it entirely
    for n in NAMES:
        rm, cs = orc.rel_max(g_cu[n], g_ref[n]), orc.cosine(g_cu[n], g_ref[n])
        assert rm <= 3e-2 and cs >= 0.999, f"grad {n}: rel_max={rm:.3e} cos={cs:.6f}"
    # and the seed matters: dropping the weight terms changes the k gradient substantially
    leaves = {n: i[n].cuda().clone().requires_grad_(True) for n in NAMES}
    o, *_ = lb.ar_fast_weight_swish_glu_weight_norm_mini_batch(*[leaves[n] for n in NAMES], 1.0, mini_batch_size=mb,
                                                               update_every=mb, use_moun=False)
    (o.float() * dO.cuda().float()).sum().backward()
    assert orc.rel_max(leaves["k"].grad.float().cpu(), g_ref["k"]) > 0.1


def test_tokens_no_apply_covers_are_zero(lb, orc):
    """ar_fast_weight_swish_glu_weight_norm_mini_batch(update_length < L): the reference writes into
    torch.zeros_like(q) and never touches the tail."""
    B, L, D, H = 1, 512, 64, 64
    i = _inputs(orc, B, L, D, H, seed=5)
    c = {k: v.cuda() for k, v in i.items()}
    kw = dict(mini_batch_size=128, update_length=256, update_every=128, use_moun=False)
    ref = orc.ar_mini_batch(*[i[n].float() for n in NAMES], 1.0, **kw)[0]
    # poison the allocator's free memory so that an uninitialised tail cannot be zero by luck
    junk = torch.full((B, L, D), 7.0, dtype=BF16, device="cuda")
    del junk
    got = lb.ar_fast_weight_swish_glu_weight_norm_mini_batch(*[c[n] for n in NAMES], 1.0, **kw)[0]
    lb.synchronize_and_check()
    assert torch.count_nonzero(ref[:, 256:]) == 0
    assert torch.count_nonzero(got[:, 256:]) == 0
    assert orc.rel_max(got[:, :256].float().cpu(), ref[:, :256].float()) <= 2e-2
