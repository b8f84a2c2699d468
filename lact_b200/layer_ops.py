"""Row-wise stages of the LaCT layer around the chunk recurrence (the layer's own code,
lact_llm/lact_model/layer_lact_swiglu.py, is outside this package; these are the passes over
[b, s, n_h * d] that sit directly on the recurrence's inputs)."""
from __future__ import annotations

import torch

from . import _lib as L

BF16 = torch.bfloat16


def _rows(t: torch.Tensor, name: str) -> torch.Tensor:
    """[b, s, n] bf16 with a contiguous last axis and 16-byte aligned rows; anything else is copied."""
    assert t.dim() == 3 and t.dtype == BF16, f"{name}: expected a [b, s, n_heads * d] bf16 tensor"
    if t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def qkv_prologue(xq: torch.Tensor, xk: torch.Tensor, xv: torch.Tensor, num_heads: int, qkv_silu: bool = True,
                 no_v_silu: bool = False):
    """fast_q, fast_k, fast_v of layer_lact_swiglu.py:399-414 (the `ttt_nope` branch) in one pass:
    `[b, s, (n_h d)] -> [(b n_h), s, d]`, SiLU on q, k (and v unless `no_v_silu`), per-head l2_norm of q and k
    (ttt_operation.py:19-26).  Inputs may be views of a fused projection."""
    if not (xq.is_cuda and xk.is_cuda and xv.is_cuda):
        raise ValueError("qkv_prologue needs CUDA tensors (there is no CPU implementation)")
    xq, xk, xv = _rows(xq, "xq"), _rows(xk, "xk"), _rows(xv, "xv")
    assert xq.shape == xk.shape == xv.shape
    b, s, nd = xq.shape
    assert nd % num_heads == 0
    d = nd // num_heads
    q, k, v = (torch.empty(b * num_heads, s, d, dtype=BF16, device=xq.device) for _ in range(3))
    with torch.cuda.device(xq.device):
        L.check(L.lib().lact_qkv_prologue(xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), xq.stride(1), xk.stride(1),
                                          xv.stride(1), xq.stride(0), xk.stride(0), xv.stride(0), q.data_ptr(),
                                          k.data_ptr(), v.data_ptr(), b, s, num_heads, d, int(bool(qkv_silu)),
                                          int(not no_v_silu), L.stream_ptr()), "lact_qkv_prologue")
    return q, k, v
