"""The allocation-free SwiGLU-FFN entry point (scratch inside the library image) against the
workspace-based entry point and the CPU oracle, through the C ABI, on two calls in a row; its
status reader; and its size limit, at exactly the limit and one step beyond.

Collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.  It passes alone in a fresh process and after the other tests.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _inputs(B, N, D, H, seed):
    g = torch.Generator().manual_seed(seed)
    w02 = (torch.randn(B, 2 * H, D, generator=g) / D ** 0.5).to(BF16).cuda()
    w1 = (torch.randn(B, D, H, generator=g) / H ** 0.5).to(BF16).cuda()
    x = torch.randn(B, N, D, generator=g).to(BF16).cuda()
    return w02, w1, x


def _lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    from lact_b200 import _lib
    return _lib.lib()


def test_static_scratch_entry_point_matches_workspace_entry_point():
    lib = _lib()
    from oracle import lact_oracle as orc
    stream = torch.cuda.current_stream().cuda_stream
    limit = lib.lact_static_scratch_bytes()
    assert limit == 16 << 20
    # two calls in a row with different shapes and data: the second call reuses the array that
    # still holds the first call's hidden activations
    for call, (B, N, D, H) in enumerate([(2, 1000, 128, 256), (3, 517, 64, 128)]):
        w02, w1, x = _inputs(B, N, D, H, seed=10 + call)
        # existing entry point (caller-provided workspace)
        need = C.c_size_t(0)
        assert lib.lact_swiglu_ffn_workspace_bytes(B, N, D, H, C.byref(need)) == 0
        ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        ref = torch.empty(B, N, D, dtype=BF16, device="cuda")
        rc = lib.lact_swiglu_ffn_fwd(w02.data_ptr(), w1.data_ptr(), x.data_ptr(), ref.data_ptr(), B, N, D, H,
                                     ws.data_ptr(), ws.numel(), stream)
        assert rc == 0
        assert lib.lact_read_status(ws.data_ptr(), stream) == 0
        # new entry point: inputs and output only
        out = torch.full((B, N, D), float("nan"), dtype=BF16, device="cuda")
        rc = lib.lact_swiglu_ffn_fwd_static(w02.data_ptr(), w1.data_ptr(), x.data_ptr(), out.data_ptr(), B, N, D, H,
                                            stream)
        assert rc == 0, lib.lact_error_string(rc)
        # the status word lives at the head of the static array: its own reader, before the next static call
        assert lib.lact_static_status(stream) == 0
        assert torch.isfinite(out.float()).all()
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert err <= 5e-3, (call, err)  # the tolerance of the SwiGLU-FFN parity test; in practice 0
        # and against the CPU restatement of the reference's fused apply (lact_swiglu_ffn.py:104-116)
        want = orc.apply_fused(w02.cpu(), w1.cpu(), x.cpu()).float()
        err = float((out.float().cpu() - want).abs().max() / want.abs().max())
        assert err <= 2e-2, (call, err)


def test_static_scratch_limit_is_exactly_what_the_header_says():
    """256 + B * N * H * 2 bytes must fit in the array: a problem that needs exactly all of it runs,
    one more token is refused (and enqueues nothing)."""
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    limit = lib.lact_static_scratch_bytes()
    B, D, H = 1, 16, 16
    N = (limit - 256) // (B * H * 2)
    assert 256 + B * N * H * 2 == limit
    w02, w1, x = _inputs(B, N, D, H, seed=12)
    out = torch.full((B, N, D), float("nan"), dtype=BF16, device="cuda")
    rc = lib.lact_swiglu_ffn_fwd_static(w02.data_ptr(), w1.data_ptr(), x.data_ptr(), out.data_ptr(), B, N, D, H, stream)
    assert rc == 0, lib.lact_error_string(rc)
    assert lib.lact_static_status(stream) == 0
    # spot-check rows at both ends and in the middle against plain fp32 arithmetic on the same bf16 values
    rows = torch.tensor([0, 1, N // 2, N - 2, N - 1], device="cuda")
    xs = x[0, rows].float()
    y = xs @ w02[0].float().t()
    hid = (torch.nn.functional.silu(y[:, :H]) * y[:, H:]).to(BF16).float()
    want = hid @ w1[0].float().t()
    err = float((out[0, rows].float() - want).abs().max() / want.abs().max())
    assert err <= 2e-2, err
    assert torch.isfinite(out.float()).all()
    # one token more: refused with the entry point's own code, and the output buffer is left alone
    out2 = torch.full((B, 8, D), 3.0, dtype=BF16, device="cuda")
    rc = lib.lact_swiglu_ffn_fwd_static(w02.data_ptr(), w1.data_ptr(), x.data_ptr(), out2.data_ptr(), B, N + 1, D, H,
                                        stream)
    assert rc == -9
    assert b"static buffer" in lib.lact_error_string(rc)
    torch.cuda.synchronize()
    assert bool((out2 == 3.0).all())
    # far beyond the limit: the same refusal
    assert lib.lact_swiglu_ffn_fwd_static(w02.data_ptr(), w1.data_ptr(), x.data_ptr(), out2.data_ptr(), 8, 4096, 64, 512,
                                          stream) == -9
