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


def lr_prologue(lr_proj: torch.Tensor, num_heads: int, base_lr: float, momentum_logits: torch.Tensor = None):
    """fw_lr1, fw_lr2, fw_lr3 (and momentum) of layer_lact_swiglu.py:463-480: softplus(lr_proj.float() +
    inv_softplus(base_lr)) split per head into three fp32 [(b n_h), s, 1] tensors; `momentum_logits` is the output of
    the momentum Linear BEFORE its Sigmoid ([b, s, n_h]); the result is sigmoid(.) in the logits' dtype, as float."""
    import math
    if not lr_proj.is_cuda:
        raise ValueError("lr_prologue needs CUDA tensors (there is no CPU implementation)")
    assert lr_proj.dim() == 3 and lr_proj.shape[2] == 3 * num_heads
    b, s, _ = lr_proj.shape

    def rows(t):
        if t.stride(2) != 1 or t.stride(0) != s * t.stride(1):
            t = t.contiguous()
        return t

    lr_proj = rows(lr_proj)
    base_lr_inv = base_lr + math.log(-math.expm1(-base_lr))
    outs = [torch.empty(b * num_heads, s, 1, dtype=torch.float32, device=lr_proj.device) for _ in range(3)]
    mom = None
    lg_ptr, lg_code, lg_ld = None, L.LACT_F32, 0
    if momentum_logits is not None:
        assert momentum_logits.shape == (b, s, num_heads)
        momentum_logits = rows(momentum_logits)
        mom = torch.empty(b * num_heads, s, 1, dtype=torch.float32, device=lr_proj.device)
        lg_ptr, lg_code, lg_ld = momentum_logits.data_ptr(), L.dtype_code(momentum_logits), momentum_logits.stride(1)
    with torch.cuda.device(lr_proj.device):
        L.check(L.lib().lact_lr_prologue(lr_proj.data_ptr(), L.dtype_code(lr_proj), lr_proj.stride(1), float(base_lr_inv),
                                         lg_ptr, lg_code, lg_ld, outs[0].data_ptr(), outs[1].data_ptr(),
                                         outs[2].data_ptr(), mom.data_ptr() if mom is not None else None, b, s, num_heads,
                                         L.stream_ptr()), "lact_lr_prologue")
    return outs[0], outs[1], outs[2], mom


def out_epilogue(fw_x: torch.Tensor, norm_weight: torch.Tensor, num_heads: int, scale_proj: torch.Tensor = None,
                 o: torch.Tensor = None, eps: float = 1e-5) -> torch.Tensor:
    """`o + merge_heads(ttt_norm(fw_x) * silu(scale_proj))` of layer_lact_swiglu.py:556-568 in one pass.
    fw_x: [(b n_h), s, d] bf16 (output of the recurrence); norm_weight: [d]; scale_proj (the output of
    `ttt_scale_proj`, before its SiLU) and o (attention output): [b, s, n_h * d] bf16 or None."""
    if not fw_x.is_cuda:
        raise ValueError("out_epilogue needs CUDA tensors (there is no CPU implementation)")
    assert fw_x.dim() == 3 and fw_x.dtype == BF16 and fw_x.shape[0] % num_heads == 0
    fw_x = fw_x.contiguous()
    B, s, d = fw_x.shape
    b = B // num_heads
    w = norm_weight.detach().float().contiguous()
    assert w.shape == (d,)

    def rows(t, name):
        assert t.shape == (b, s, num_heads * d), f"{name}: expected [b, s, n_heads * d]"
        t = _rows(t, name)
        return t if t.stride(0) == s * t.stride(1) else t.contiguous()

    gate = rows(scale_proj, "scale_proj") if scale_proj is not None else None
    res = rows(o, "o") if o is not None else None
    out = torch.empty(b, s, num_heads * d, dtype=BF16, device=fw_x.device)
    with torch.cuda.device(fw_x.device):
        L.check(L.lib().lact_out_epilogue(fw_x.data_ptr(), w.data_ptr(), gate.data_ptr() if gate is not None else None,
                                          gate.stride(1) if gate is not None else 0,
                                          res.data_ptr() if res is not None else None,
                                          res.stride(1) if res is not None else 0, out.data_ptr(), out.stride(1), b, s,
                                          num_heads, d, float(eps), L.stream_ptr()), "lact_out_epilogue")
    return out

