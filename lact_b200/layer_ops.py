"""Row-wise stages of the LaCT layer around the chunk recurrence (the layer's own code,
lact_llm/lact_model/layer_lact_swiglu.py, is outside this package; these are the passes over
[b, s, n_h * d] that sit directly on the recurrence's inputs and output).

Forward: one fused CUDA pass each.  Backward (training): each pass is an autograd Function; the two passes over
[b, s, n_h * d] (`qkv_prologue`, `out_epilogue`) have fused backward kernels that recompute from the saved inputs
(the forward's bf16 roundings are treated as identities); the small learning-rate pass differentiates a plain
PyTorch restatement.

Attention half of the hybrid layers (tcgen05 kernels, forward and backward, head dimension 64 or 128):
`sliding_window_attention` (causal band; packed sequences by `cu_seqlens`, padded batches by `attention_mask`),
`block_attention` (not causal, own key count) and, under the reference's names, the autoregressive-video layer's
`batched_sliding_window_attention`, `batched_sliding_window_attention_with_repeated_chunks` and
`sliding_window_attention_inference`."""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib as L

BF16 = torch.bfloat16


def _heads(t: torch.Tensor, n_h: int) -> torch.Tensor:
    b, s, nd = t.shape
    return t.reshape(b, s, n_h, nd // n_h).permute(0, 2, 1, 3).reshape(b * n_h, s, nd // n_h)


def _unheads(t: torch.Tensor, n_h: int) -> torch.Tensor:
    B, s, d = t.shape
    return t.reshape(B // n_h, n_h, s, d).permute(0, 2, 1, 3).reshape(B // n_h, s, n_h * d)


class _QkvPrologue(torch.autograd.Function):
    """Forward: the fused kernel.  Backward: `lact_qkv_prologue_bwd` on the saved projections (rotation transposed,
    l2-norm and SiLU differentiated in one pass per row)."""
    @staticmethod
    def forward(ctx, xq, xk, xv, num_heads, qkv_silu, v_silu, cos, sin, rope_hd, offset, seq_start=None):
        ctx.save_for_backward(xq, xk, xv, *((cos, sin) if cos is not None else ()))
        ctx.cfg = (num_heads, qkv_silu, v_silu, rope_hd, offset)
        ctx.seq_start = seq_start   # int32 index tensor, no gradient
        return _qkv_prologue_fwd(xq, xk, xv, num_heads, qkv_silu, v_silu, cos, sin, rope_hd, offset, seq_start)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        saved = ctx.saved_tensors
        n_h, qkv_silu, v_silu, rope_hd, offset = ctx.cfg
        xs = [_rows(t, "projection") for t in saved[:3]]
        b, s, nd = xs[0].shape
        d = nd // n_h
        cos, sin = (saved[3], saved[4]) if len(saved) == 5 else (None, None)
        dzs = [None if g is None else g.to(BF16).contiguous() for g in (dq, dk, dv)]
        outs = [torch.empty(b, s, nd, dtype=BF16, device=xs[0].device) for _ in range(3)]
        with torch.cuda.device(xs[0].device):
            L.check(L.lib().lact_qkv_prologue_bwd(
                xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), xs[0].stride(1), xs[1].stride(1), xs[2].stride(1),
                xs[0].stride(0), xs[1].stride(0), xs[2].stride(0), *[None if g is None else g.data_ptr() for g in dzs],
                outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), b, s, n_h, d, int(qkv_silu), int(v_silu),
                cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None,
                int(rope_hd) if cos is not None else 0, cos.shape[0] if cos is not None else 0, int(offset),
                ctx.seq_start.data_ptr() if ctx.seq_start is not None else None, L.stream_ptr()), "lact_qkv_prologue_bwd")
        return (*[o.to(x.dtype) for o, x in zip(outs, saved[:3])], None, None, None, None, None, None, None, None)


def _seq_start(cu_seqlens: torch.Tensor, n_tokens: int, device) -> torch.Tensor:
    """int32 [n_tokens]: for every token of a packed batch entry, the first token of its sequence (no host
    synchronisation: the output size is known)."""
    cu = cu_seqlens.to(device=device, dtype=torch.int64)
    return torch.repeat_interleave(cu[:-1], cu[1:] - cu[:-1], output_size=n_tokens).to(torch.int32).contiguous()


def _rows(t: torch.Tensor, name: str) -> torch.Tensor:
    """[b, s, n] bf16 with a contiguous last axis and 16-byte aligned rows; anything else is copied."""
    assert t.dim() == 3 and t.dtype == BF16, f"{name}: expected a [b, s, n_heads * d] bf16 tensor"
    if t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def rotary_tables(head_dim: int, n_positions: int, base: float = 500000.0, device=None, dtype=BF16):
    """cos / sin tables [n_positions, head_dim / 2] as fla.modules.RotaryEmbedding(dim=head_dim, base=rope_theta)
    caches them (fp32 inverse frequencies and positions, result cast to the activations' dtype)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    freqs = torch.outer(torch.arange(n_positions, dtype=torch.float32, device=device), inv_freq)
    return torch.cos(freqs).to(dtype), torch.sin(freqs).to(dtype)


def _qkv_prologue_fwd(xq, xk, xv, num_heads, qkv_silu, v_silu, cos, sin, rope_hd, offset, seq_start=None):
    xq, xk, xv = _rows(xq, "xq"), _rows(xk, "xk"), _rows(xv, "xv")
    b, s, nd = xq.shape
    d = nd // num_heads
    q, k, v = (torch.empty(b * num_heads, s, d, dtype=BF16, device=xq.device) for _ in range(3))
    lib = L.lib()
    with torch.cuda.device(xq.device):
        if cos is None:
            L.check(lib.lact_qkv_prologue(xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), xq.stride(1), xk.stride(1),
                                          xv.stride(1), xq.stride(0), xk.stride(0), xv.stride(0), q.data_ptr(),
                                          k.data_ptr(), v.data_ptr(), b, s, num_heads, d, int(bool(qkv_silu)),
                                          int(bool(v_silu)), L.stream_ptr()), "lact_qkv_prologue")
        else:
            L.check(lib.lact_qkv_prologue_rope(xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), xq.stride(1), xk.stride(1),
                                               xv.stride(1), xq.stride(0), xk.stride(0), xv.stride(0), q.data_ptr(),
                                               k.data_ptr(), v.data_ptr(), b, s, num_heads, d, int(bool(qkv_silu)),
                                               int(bool(v_silu)), cos.data_ptr(), sin.data_ptr(), int(rope_hd),
                                               cos.shape[0], int(offset),
                                               seq_start.data_ptr() if seq_start is not None else None,
                                               L.stream_ptr()), "lact_qkv_prologue_rope")
    return q, k, v


def qkv_prologue(xq: torch.Tensor, xk: torch.Tensor, xv: torch.Tensor, num_heads: int, qkv_silu: bool = True,
                 no_v_silu: bool = False, rotary: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None,
                 seqlen_offset: int = 0, cu_seqlens: Optional[torch.Tensor] = None):
    """fast_q, fast_k, fast_v of layer_lact_swiglu.py:399-446 in one pass: `[b, s, (n_h d)] -> [(b n_h), s, d]`, SiLU
    on q, k (and v unless `no_v_silu`), per-head l2_norm of q and k (ttt_operation.py:19-26) and, when `rotary` =
    (cos, sin, attention_head_dim) is given (`ttt_nope` off), the rotary embedding of q and k over attention heads of
    that size (tables as `rotary_tables` / fla.modules.RotaryEmbedding build them, bf16 [positions, head_dim / 2]).
    Inputs may be views of a fused projection.  Differentiable (see the module docstring).  `cu_seqlens` (with
    `rotary`, batch of one): sequences packed back to back, positions restart at every sequence start (:434)."""
    if not (xq.is_cuda and xk.is_cuda and xv.is_cuda):
        raise ValueError("qkv_prologue needs CUDA tensors (there is no CPU implementation)")
    assert xq.shape == xk.shape == xv.shape and xq.dim() == 3 and xq.shape[2] % num_heads == 0
    cos = sin = None
    rope_hd = 0
    if rotary is not None:
        cos, sin, rope_hd = rotary
        assert cos.dtype == BF16 and sin.dtype == BF16 and cos.shape == sin.shape and cos.shape[1] * 2 == rope_hd
        cos, sin = cos.contiguous(), sin.contiguous()
    seq_start = None
    if cu_seqlens is not None and rotary is not None:
        if xq.shape[0] != 1:
            raise ValueError("packed sequences (cu_seqlens) need a batch of one")
        seq_start = _seq_start(cu_seqlens, xq.shape[1], xq.device)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (xq, xk, xv)):
        return _QkvPrologue.apply(xq, xk, xv, num_heads, bool(qkv_silu), not no_v_silu, cos, sin, int(rope_hd),
                                  int(seqlen_offset), seq_start)
    return _qkv_prologue_fwd(xq, xk, xv, num_heads, bool(qkv_silu), not no_v_silu, cos, sin, int(rope_hd),
                             int(seqlen_offset), seq_start)


class _LrPrologue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lr_proj, momentum_logits, num_heads, base_lr):
        ctx.save_for_backward(lr_proj, *((momentum_logits,) if momentum_logits is not None else ()))
        ctx.cfg = (num_heads, base_lr)
        outs = _lr_prologue_fwd(lr_proj, num_heads, base_lr, momentum_logits)
        return outs if outs[3] is not None else (outs[0], outs[1], outs[2])

    @staticmethod
    def backward(ctx, *grads):
        saved = ctx.saved_tensors
        n_h, base_lr = ctx.cfg
        base_lr_inv = base_lr + math.log(-math.expm1(-base_lr))
        with torch.enable_grad():
            p = saved[0].detach().float().requires_grad_(True)
            lr = _heads(F.softplus(p + base_lr_inv), n_h)  # [(b n_h), s, 3]
            outs, leaves = [lr[..., i:i + 1] for i in range(3)], [p]
            if len(saved) == 2:
                m = saved[1].detach().float().requires_grad_(True)
                outs.append(_heads(torch.sigmoid(m), n_h))
                leaves.append(m)
            g = torch.autograd.grad(outs, leaves, [gi.float() for gi in grads[:len(outs)]])
        gm = g[1].to(saved[1].dtype) if len(saved) == 2 else None
        return g[0].to(saved[0].dtype), gm, None, None


def lr_prologue(lr_proj: torch.Tensor, num_heads: int, base_lr: float, momentum_logits: torch.Tensor = None):
    """fw_lr1, fw_lr2, fw_lr3 (and momentum) of layer_lact_swiglu.py:463-480; see `_lr_prologue_fwd`.  Differentiable
    with respect to the projections (see the module docstring)."""
    if torch.is_grad_enabled() and (lr_proj.requires_grad or (momentum_logits is not None and momentum_logits.requires_grad)):
        outs = _LrPrologue.apply(lr_proj, momentum_logits, num_heads, float(base_lr))
        return (outs[0], outs[1], outs[2], outs[3] if len(outs) == 4 else None)
    return _lr_prologue_fwd(lr_proj, num_heads, base_lr, momentum_logits)


def _lr_prologue_fwd(lr_proj: torch.Tensor, num_heads: int, base_lr: float, momentum_logits: torch.Tensor = None):
    """fw_lr1, fw_lr2, fw_lr3 (and momentum) of layer_lact_swiglu.py:463-480: softplus(lr_proj.float() +
    inv_softplus(base_lr)) split per head into three fp32 [(b n_h), s, 1] tensors; `momentum_logits` is the output of
    the momentum Linear BEFORE its Sigmoid ([b, s, n_h]); the result is sigmoid(.) in the logits' dtype, as float."""
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


class _OutEpilogue(torch.autograd.Function):
    """Forward: the fused kernel.  Backward: `lact_out_epilogue_bwd` (RMSNorm, gate and head merge differentiated in
    one pass per row; the norm weight's gradient as per-block partial sums added here)."""
    @staticmethod
    def forward(ctx, fw_x, norm_weight, scale_proj, o, num_heads, eps):
        ctx.save_for_backward(fw_x, norm_weight, *((scale_proj,) if scale_proj is not None else ()))
        ctx.cfg = (num_heads, eps, scale_proj is not None, o is not None)
        return _out_epilogue_fwd(fw_x, norm_weight, num_heads, scale_proj, o, eps)

    @staticmethod
    def backward(ctx, dout):
        saved = ctx.saved_tensors
        n_h, eps, has_gate, has_o = ctx.cfg
        x = saved[0].contiguous()
        B, s, d = x.shape
        b = B // n_h
        w = saved[1].detach().float().contiguous()
        gate = None
        if has_gate:
            gate = _rows(saved[2], "scale_proj")
            gate = gate if gate.stride(0) == s * gate.stride(1) else gate.contiguous()
        dy = _rows(dout.to(BF16), "grad")
        dy = dy if dy.stride(0) == s * dy.stride(1) else dy.contiguous()
        dx = torch.empty_like(x)
        dgate = torch.empty(b, s, n_h * d, dtype=BF16, device=x.device) if has_gate else None
        blocks = L.lib().lact_out_epilogue_bwd_blocks()
        part = torch.empty(blocks, d, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            L.check(L.lib().lact_out_epilogue_bwd(x.data_ptr(), w.data_ptr(), gate.data_ptr() if has_gate else None,
                                                  gate.stride(1) if has_gate else 0, dy.data_ptr(), dy.stride(1),
                                                  dx.data_ptr(), dgate.data_ptr() if has_gate else None, part.data_ptr(),
                                                  b, s, n_h, d, float(eps), L.stream_ptr()), "lact_out_epilogue_bwd")
        dw = part.sum(dim=0).to(saved[1].dtype)
        return (dx.to(saved[0].dtype), dw, dgate.to(saved[2].dtype) if has_gate else None, dout if has_o else None,
                None, None)


def out_epilogue(fw_x: torch.Tensor, norm_weight: torch.Tensor, num_heads: int, scale_proj: torch.Tensor = None,
                 o: torch.Tensor = None, eps: float = 1e-5) -> torch.Tensor:
    """`o + merge_heads(ttt_norm(fw_x) * silu(scale_proj))` of layer_lact_swiglu.py:556-568 in one pass; see
    `_out_epilogue_fwd`.  Differentiable with respect to fw_x, the norm weight, scale_proj and o (module docstring)."""
    ts = [t for t in (fw_x, norm_weight, scale_proj, o) if t is not None]
    if torch.is_grad_enabled() and any(t.requires_grad for t in ts):
        return _OutEpilogue.apply(fw_x, norm_weight, scale_proj, o, num_heads, float(eps))
    return _out_epilogue_fwd(fw_x, norm_weight, num_heads, scale_proj, o, eps)


def _out_epilogue_fwd(fw_x: torch.Tensor, norm_weight: torch.Tensor, num_heads: int, scale_proj: torch.Tensor = None,
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



# ------------------------------------------------------------------------------------------ sliding-window attention
def _head_view(t: torch.Tensor, h: int, d: int) -> torch.Tensor:
    """[b, l, h, d] with heads adjacent within a token and 16-byte aligned token / batch strides (the layout of a slice
    of a fused projection reshaped to heads); anything else is copied."""
    if (t.stride(3) != 1 or t.stride(2) != d or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16
            or t.stride(1) < h * d):
        t = t.contiguous()
    return t


@torch.library.custom_op("lact_b200::swa_fwd", mutates_args=(), device_types="cuda")
def _swa_fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, softmax_scale: float,
                seq_start: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """[o, lse]: the attention output and every row's log-sum-exp (log2 domain, fp32 [b, h, l]) for the backward.
    window > 0: causal, the last `window` keys; 0: causal, all earlier keys; < 0: block attention (not causal: every
    query sees all keys of its batch entry; k and v may then hold another number of tokens than q)."""
    from .backward import _status_word, post_status, reset_status
    b, l, h, d = q.shape
    lk = k.shape[1]
    q, k, v = _head_view(q, h, d), _head_view(k, h, d), _head_view(v, h, d)
    o = torch.empty(b, l, h, d, dtype=BF16, device=q.device)
    lse = torch.empty(b, h, l, dtype=torch.float32, device=q.device)
    reset_status(q.device)
    with torch.cuda.device(q.device):
        L.check(L.lib().lact_swa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), b, l, lk, h, d, q.stride(1),
                                     q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0), o.stride(1),
                                     o.stride(0), int(window), float(softmax_scale),
                                     seq_start.data_ptr() if seq_start is not None else None, lse.data_ptr(),
                                     _status_word(q.device).data_ptr(), L.stream_ptr()), "lact_swa_fwd")
    post_status(q.device)
    return [o, lse]


@_swa_fwd_op.register_fake
def _swa_fwd_fake(q, k, v, window, softmax_scale, seq_start=None):
    b, l, h, d = q.shape
    return [q.new_empty(q.shape), q.new_empty((b, h, l), dtype=torch.float32)]


@torch.library.custom_op("lact_b200::swa_bwd", mutates_args=(), device_types="cuda")
def _swa_bwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                dout: torch.Tensor, window: int, softmax_scale: float,
                seq_start: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """[dq, dk, dv] (bf16, contiguous): probabilities recomputed from lse, five products per (query tile, key tile)."""
    from .backward import _status_word, post_status, reset_status
    b, l, h, d = q.shape
    lk = k.shape[1]
    q, k, v = _head_view(q, h, d), _head_view(k, h, d), _head_view(v, h, d)
    o, dout = _head_view(o, h, d), _head_view(dout.to(BF16), h, d)
    dq = torch.empty(b, l, h, d, dtype=BF16, device=q.device)
    dk, dv = (torch.empty(b, lk, h, d, dtype=BF16, device=q.device) for _ in range(2))
    delta = torch.empty(b, h, l, dtype=torch.float32, device=q.device)
    reset_status(q.device)
    with torch.cuda.device(q.device):
        L.check(L.lib().lact_swa_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(),
                                     lse.contiguous().data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                     delta.data_ptr(), b, l, lk, h, d, q.stride(1), q.stride(0), k.stride(1), k.stride(0),
                                     v.stride(1), v.stride(0), o.stride(1), o.stride(0), dout.stride(1), dout.stride(0),
                                     int(window), float(softmax_scale),
                                     seq_start.data_ptr() if seq_start is not None else None,
                                     _status_word(q.device).data_ptr(), L.stream_ptr()), "lact_swa_bwd")
    post_status(q.device)
    return [dq, dk, dv]


@_swa_bwd_op.register_fake
def _swa_bwd_fake(q, k, v, o, lse, dout, window, softmax_scale, seq_start=None):
    return [q.new_empty(q.shape), q.new_empty(k.shape), q.new_empty(k.shape)]


def _swa_setup(ctx, inputs, output):
    q, k, v, window, scale, seq_start = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1], *((seq_start,) if seq_start is not None else ()))
    ctx.cfg = (int(window), float(scale))
    ctx.set_materialize_grads(False)


def _swa_autograd(ctx, grads):
    q, k, v, o, lse = ctx.saved_tensors[:5]
    seq_start = ctx.saved_tensors[5] if len(ctx.saved_tensors) == 6 else None
    dout = grads[0]
    # one entry per input the caller passed: an omitted (None) seq_start is not an input of the autograd node
    tail = (None, None, None) if seq_start is not None else (None, None)
    if dout is None:
        return (None, None, None) + tail
    dq, dk, dv = torch.ops.lact_b200.swa_bwd(q, k, v, o, lse, dout.contiguous(), ctx.cfg[0], ctx.cfg[1], seq_start)
    return (dq, dk, dv) + tail


_swa_fwd_op.register_autograd(_swa_autograd, setup_context=_swa_setup)


def sliding_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window_size: Optional[int] = None,
                             softmax_scale: Optional[float] = None,
                             cu_seqlens: Optional[torch.Tensor] = None,
                             attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention over the last `window_size` keys (the query's own position included), q, k, v and the
    result [b, l, n_heads, head_dim] bf16: what `flash_attn_func(q, k, v, causal=True, window_size=(window_size - 1,
    0))` computes at lact_llm/lact_model/layer_lact_swiglu.py:386-394 and
    minimal_implementations/causal_lact_with_sliding_window_attn.py:380-384 (`window_size=None`: all earlier keys).
    head_dim 64 or 128.  Differentiable (dq, dk, dv by `lact_swa_bwd`).  `cu_seqlens` (int32 [n + 1], device): the batch
    entry (b must be 1) is n sequences packed back to back, as for `flash_attn_varlen_func` (:371-385): no query sees
    a key of an earlier sequence.  `attention_mask` ([b, l], nonzero = token, zero = padding, any padding side): the
    padded-batch branch (:351-370): the real tokens of all entries are gathered into one packed entry, attended per
    sequence and scattered back, padding positions of the result are zero (`unpad_input` / `pad_input`).  Like the
    reference's, this branch reads the number of real tokens on the host."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("sliding_window_attention needs CUDA tensors (there is no CPU implementation)")
    assert q.dim() == 4 and q.shape == k.shape == v.shape, "q, k, v: [b, l, n_heads, head_dim], equal head counts"
    assert q.dtype == k.dtype == v.dtype == BF16, "bf16 activations"
    if q.shape[3] not in (64, 128):
        raise ValueError("head_dim must be 64 or 128")
    scale = float(softmax_scale) if softmax_scale is not None else q.shape[3] ** -0.5
    window = int(window_size) if window_size else 0
    if attention_mask is not None:
        if cu_seqlens is not None:
            raise ValueError("give attention_mask or cu_seqlens, not both")
        b, l, h, d = q.shape
        assert attention_mask.shape == (b, l), "attention_mask: [b, l]"
        mask = attention_mask.to(device=q.device) != 0
        idx = torch.nonzero(mask.reshape(-1)).reshape(-1)   # (host synchronisation: data-dependent size)
        if idx.numel() == 0:
            return torch.zeros_like(q)
        cu = torch.nn.functional.pad(torch.cumsum(mask.sum(dim=1), 0), (1, 0)).to(torch.int32)
        packed = [t.reshape(b * l, h, d).index_select(0, idx).unsqueeze(0) for t in (q, k, v)]
        o = torch.ops.lact_b200.swa_fwd(*packed, window, scale, _seq_start(cu, idx.numel(), q.device))[0]
        return torch.zeros(b * l, h, d, dtype=q.dtype, device=q.device).index_copy(0, idx, o[0]).reshape(b, l, h, d)
    seq_start = None
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError("packed sequences (cu_seqlens) need a batch of one")
        seq_start = _seq_start(cu_seqlens, q.shape[1], q.device)
    return torch.ops.lact_b200.swa_fwd(q, k, v, window, scale, seq_start)[0]


def block_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Full (not causal) attention of every query of a batch entry over all keys of that entry: q [b, lq, h, d],
    k, v [b, lk, h, d] bf16, result [b, lq, h, d].  What `flash_attention(q, k, v, k_lens=<all keys>, window_size=(-1,
    -1))` computes for the frame blocks of the autoregressive-video layer
    (lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:313-318, 344-364).  The same tcgen05 kernels as
    `sliding_window_attention`, band and sequence masks off.  head_dim 64 or 128.  Differentiable."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("block_attention needs CUDA tensors (there is no CPU implementation)")
    assert q.dim() == 4 and k.shape == v.shape and k.dim() == 4, "q [b, lq, h, d]; k, v [b, lk, h, d]"
    assert q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:], "q and k, v differ in the token count only"
    assert q.dtype == k.dtype == v.dtype == BF16, "bf16 activations"
    if q.shape[3] not in (64, 128):
        raise ValueError("head_dim must be 64 or 128")
    if q.shape[1] == 0 or k.shape[1] == 0:
        return torch.zeros_like(q)
    scale = float(softmax_scale) if softmax_scale is not None else q.shape[3] ** -0.5
    return torch.ops.lact_b200.swa_fwd(q, k, v, -1, scale, None)[0]


def batched_sliding_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mini_batch_size: int,
                                     update_every: int, num_chunks: int, kv_cache_size: int) -> torch.Tensor:
    """The block attention of the autoregressive-video layer, same name and arguments as
    ar_lact_swa_repeat.py:299-365.  q, k, v: [b, l, h, d] with l = update_every - mini_batch_size + update_every *
    (num_chunks - 1).  The first update_every - mini_batch_size tokens attend among themselves; every later block of
    update_every tokens is a clean part (the first mini_batch_size tokens, attending among themselves) followed by a
    noisy part that attends over the last kv_cache_size clean keys and the keys after them (mini_batch_size +
    kv_cache_size keys, as the reference's k_lens says)."""
    b, l = q.shape[:2]
    first, n_c, mb = update_every - mini_batch_size, num_chunks - 1, mini_batch_size
    assert l == first + update_every * n_c, "l = update_every - mini_batch_size + update_every * (num_chunks - 1)"
    assert 0 <= kv_cache_size <= mb
    parts = [block_attention(q[:, :first], k[:, :first], v[:, :first])] if first > 0 else []
    if n_c > 0:
        q_r, k_r, v_r = (t[:, first:].reshape(b * n_c, update_every, *t.shape[2:]) for t in (q, k, v))
        o_clean = block_attention(q_r[:, :mb], k_r[:, :mb], v_r[:, :mb])
        k_end = min(update_every, 2 * mb)   # keys [mb - kv_cache_size, mb - kv_cache_size + (mb + kv_cache_size))
        o_noise = block_attention(q_r[:, mb:], k_r[:, mb - kv_cache_size:k_end], v_r[:, mb - kv_cache_size:k_end])
        parts.append(torch.cat([o_clean, o_noise], dim=1).reshape(b, n_c * update_every, *q.shape[2:]))
    return torch.cat(parts, dim=1) if len(parts) > 1 else parts[0]


def batched_sliding_window_attention_with_repeated_chunks(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                                          mini_batch_size: int, update_every: int, num_chunks: int,
                                                          kv_cache_size: int) -> torch.Tensor:
    """ar_lact_swa_repeat.py:368-463, same name and arguments: update_every = (num_repeat + 1) * mini_batch_size.  The
    first update_every - mini_batch_size tokens are num_repeat blocks of mini_batch_size tokens, each attending within
    itself; every later block of update_every tokens is a clean part (mini_batch_size tokens, attending within itself)
    and num_repeat noisy parts, each attending over the last kv_cache_size clean keys and its own keys."""
    b, l = q.shape[:2]
    first, n_c, mb = update_every - mini_batch_size, num_chunks - 1, mini_batch_size
    nr = update_every // mb - 1
    assert update_every == (nr + 1) * mb and nr >= 1, "update_every must be a multiple (>= 2) of mini_batch_size"
    assert l == first + update_every * n_c and 0 <= kv_cache_size <= mb
    tail = q.shape[2:]
    blocks = lambda t: t[:, :first].reshape(b * nr, mb, *tail)
    parts = [block_attention(blocks(q), blocks(k), blocks(v)).reshape(b, first, *tail)]
    if n_c > 0:
        q_r, k_r, v_r = (t[:, first:].reshape(b * n_c, update_every, *tail) for t in (q, k, v))
        o_clean = block_attention(q_r[:, :mb], k_r[:, :mb], v_r[:, :mb])
        noisy = lambda t: t[:, mb:].reshape(b * n_c * nr, mb, *tail)
        cached = lambda t: t[:, mb - kv_cache_size:mb].repeat_interleave(nr, dim=0)
        o_noise = block_attention(noisy(q_r), torch.cat([cached(k_r), noisy(k_r)], dim=1),
                                  torch.cat([cached(v_r), noisy(v_r)], dim=1)).reshape(b * n_c, nr * mb, *tail)
        parts.append(torch.cat([o_clean, o_noise], dim=1).reshape(b, n_c * update_every, *tail))
    return torch.cat(parts, dim=1) if len(parts) > 1 else parts[0]


def sliding_window_attention_inference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mini_batch_size: int,
                                       kv_cache: Optional[torch.Tensor] = None, interleave: bool = False,
                                       kv_cache_size: int = 1560) -> torch.Tensor:
    """ar_lact_swa_repeat.py:464-531, same name and arguments: the attention of one generation step of the
    autoregressive-video layer.  (1) no cache, not interleaved: full attention; (2) interleaved: the first
    mini_batch_size (clean) tokens attend among themselves, the rest over the last kv_cache_size clean keys and their
    own; (3) with a cache ([2 b, l_c, h, d]: keys of all entries, then values): full attention over cache + k."""
    if kv_cache is None and not interleave:
        return block_attention(q, k, v)
    if interleave:
        mb = mini_batch_size
        o_clean = block_attention(q[:, :mb], k[:, :mb], v[:, :mb])
        o_rest = block_attention(q[:, mb:], k[:, mb - kv_cache_size:], v[:, mb - kv_cache_size:])
        return torch.cat([o_clean, o_rest], dim=1)
    k_cache, v_cache = kv_cache.chunk(2, dim=0)
    return block_attention(q, torch.cat([k_cache, k], dim=1), torch.cat([v_cache, v], dim=1))
