"""The allocation-free SwiGLU-FFN entry point (scratch inside the library image) against the
workspace-based entry point, through the C ABI, on two calls in a row.

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


def test_static_scratch_entry_point_matches_workspace_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    from lact_b200 import _lib
    lib = _lib.lib()
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
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert err <= 5e-3, (call, err)  # the tolerance of the SwiGLU-FFN parity test; in practice 0
    # a problem whose hidden activations exceed the static array is refused with its own code
    B, N, D, H = 8, 4096, 64, 512
    assert 256 + B * N * H * 2 > limit
    w02, w1, x = _inputs(1, 16, D, H, seed=3)  # pointers only need to be non-null: nothing is enqueued
    rc = lib.lact_swiglu_ffn_fwd_static(w02.data_ptr(), w1.data_ptr(), x.data_ptr(), x.data_ptr(), B, N, D, H, stream)
    assert rc == -9
    assert b"static buffer" in lib.lact_error_string(rc)
