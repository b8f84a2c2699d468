"""fp32-activation mode of the chunk recurrence (the reference's fp32 configuration, e.g.
minimal_implementations/bidirectional_lact_layer.py:73-160 called with fp32 q, k, v).

The step program is the same one `ops.scan` hands to `lact_scan_fwd`; here it is executed from
Python, one C-ABI call per contraction / pointwise plane / renorm, because the tcgen05 pipe has
no fp32 x fp32 MMA: the contractions run as plain FFMA kernels (`lact_sgemm_f32`).  This mode
exists for accuracy (about 1e-6 relative when Muon is off), not throughput.  The Newton-Schulz
step casts its input to bf16 in the reference too (ttt_operation.py:30-66), so it runs on the
tcgen05 engine as in bf16 mode.

Forward only.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib as L
from . import program as P

F32 = torch.float32
BF16 = torch.bfloat16


def _sgemm(a, a_t, b, b_t, c, M, N, K, accumulate=False, beta=None):
    """c[b] = op(a[b]) op(b[b])^T on contiguous fp32 tensors (see `lact_sgemm_f32`)."""
    assert a.is_contiguous() and b.is_contiguous() and c.is_contiguous()
    assert a.dtype == b.dtype == c.dtype == F32
    with torch.cuda.device(c.device):
        L.check(L.lib().lact_sgemm_f32(a.data_ptr(), int(a_t), b.data_ptr(), int(b_t), c.data_ptr(), int(accumulate),
                                       beta.data_ptr() if beta is not None else None, c.shape[0], M, N, K,
                                       L.stream_ptr()), "lact_sgemm_f32")


def _planes(y02, dh, lrs, w_scale, dy02, hid, rows, H):
    lr0, lr1, lr2 = lrs if lrs is not None else (None, None, None)
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(y02.device):
        L.check(L.lib().lact_swiglu_planes_f32(y02.data_ptr(), ptr(dh), ptr(lr0), ptr(lr1), ptr(lr2),
                                               L.dtype_code(lr0) if lr0 is not None else L.LACT_F32, float(w_scale),
                                               ptr(dy02), hid.data_ptr(), rows, H, L.stream_ptr()),
                "lact_swiglu_planes_f32")


def _add_renorm(master, compute, shadow, n0, g, x, mode, prenorm, prenorm_bf16, quirk):
    B, R, Cc = master.shape
    with torch.cuda.device(master.device):
        L.check(L.lib().lact_add_renorm(master.data_ptr(), compute.data_ptr() if compute is not None else None,
                                        shadow.data_ptr(), n0.data_ptr(), g.data_ptr(),
                                        x.data_ptr() if x is not None else None, B, R, Cc, int(mode), int(prenorm),
                                        int(prenorm_bf16), int(quirk), L.stream_ptr()), "lact_add_renorm")


def scan_f32(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps: Sequence[P.Step], *, out_len: Optional[int] = None,
             momentum=None, m_init=None, use_muon=False, ns_steps=5, ns_const_coeffs=False, ns_concat=False,
             ns_gram_right=False, renorm=L.RENORM_EPS_OUTSIDE, prenorm=False, prenorm_bf16=False,
             overwrite_quirk=False, w_scale=1.0, return_state=False, return_momentum=False):
    """Same arguments and results as `ops.scan`, fp32 activations in, fp32 output."""
    from .ops import zeropower_via_newtonschulz5

    dev = q.device
    B, Ltok, D = k.shape
    H = w0.shape[1]
    if D % 4 or H % 4:
        raise ValueError("fp32 mode needs head dimensions that are multiples of 4")
    q, k, v = (t.contiguous() for t in (q, k, v))
    out_len = Ltok if out_len is None else int(out_len)
    o = torch.zeros(B, out_len, D, dtype=F32, device=dev)

    # masters: W0|W2 stacked [B, 2H, D] (one contraction with the tokens), W1 [B, D, H]
    w02 = torch.cat([w0.float(), w2.float()], dim=1).contiguous()
    w1 = w1.float().contiguous().clone()
    n02 = w02.norm(dim=2).contiguous()
    n1 = w1.norm(dim=2).contiguous()
    c02 = c1 = None  # pre-norm: normalised copies the steps compute with
    if prenorm:
        c02, c1 = w02.clone(), w1.clone()
    shadow02 = torch.empty(B, 2 * H, D, dtype=BF16, device=dev)
    shadow1 = torch.empty(B, D, H, dtype=BF16, device=dev)
    m02 = m1 = None
    if momentum is not None:
        if m_init is not None:
            m02 = torch.cat([m_init[0].float(), m_init[2].float()], dim=1).contiguous()
            m1 = m_init[1].float().contiguous().clone()
        else:
            m02 = torch.zeros(B, 2 * H, D, dtype=F32, device=dev)
            m1 = torch.zeros(B, D, H, dtype=F32, device=dev)
        momentum = momentum.float()

    def weights():
        return (c02, c1) if prenorm else (w02, w1)

    for kind, s, e, out in steps:
        n = e - s
        if n <= 0:
            continue
        a02, a1 = weights()
        if kind == P.APPLY:
            x = q[:, s:e].contiguous()
            y02 = torch.empty(B, n, 2 * H, dtype=F32, device=dev)
            _sgemm(x, 0, a02, 0, y02, n, 2 * H, D)
            hid = torch.empty(B, n, H, dtype=F32, device=dev)
            _planes(y02, None, None, 1.0, None, hid, B * n, H)
            if n == out_len and out == 0:
                _sgemm(hid, 0, a1, 0, o, n, D, H)
            else:
                t = torch.empty(B, n, D, dtype=F32, device=dev)
                _sgemm(hid, 0, a1, 0, t, n, D, H)
                o[:, out:out + n].copy_(t)
            continue
        ks, vs = k[:, s:e].contiguous(), v[:, s:e].contiguous()
        lrs = tuple(t[:, s:e].contiguous() for t in (lr0, lr1, lr2))
        y02 = torch.empty(B, n, 2 * H, dtype=F32, device=dev)
        _sgemm(ks, 0, a02, 0, y02, n, 2 * H, D)
        dh = torch.empty(B, n, H, dtype=F32, device=dev)
        _sgemm(vs, 0, a1, 1, dh, n, H, D)
        dy02 = torch.empty_like(y02)
        hid = torch.empty_like(dh)
        _planes(y02, dh, lrs, w_scale, dy02, hid, B * n, H)
        if momentum is not None:
            # G = dW + mean(beta) * M, written over M (ttt_operation.py:170-181)
            beta = momentum[:, s:e].mean(dim=1).contiguous()
            g02, g1 = m02, m1
            _sgemm(dy02, 1, ks, 1, g02, 2 * H, D, n, accumulate=True, beta=beta)
            _sgemm(vs, 1, hid, 1, g1, D, H, n, accumulate=True, beta=beta)
        else:
            g02 = torch.empty(B, 2 * H, D, dtype=F32, device=dev)
            g1 = torch.empty(B, D, H, dtype=F32, device=dev)
            _sgemm(dy02, 1, ks, 1, g02, 2 * H, D, n)
            _sgemm(vs, 1, hid, 1, g1, D, H, n)
        x02 = x1 = None
        if use_muon:
            st = int(ns_steps) if ns_const_coeffs else None

            def ns(g):
                if ns_gram_right:  # NVS layout: the matrix is stored transposed (lact_nvs/lact_ttt.py:32-67)
                    return zeropower_via_newtonschulz5(g.transpose(1, 2).contiguous(), st).transpose(1, 2).contiguous()
                return zeropower_via_newtonschulz5(g, st)

            x1 = ns(g1)
            x02 = ns(g02) if ns_concat else torch.cat([ns(g02[:, :H]), ns(g02[:, H:])], dim=1)
        _add_renorm(w02, c02, shadow02, n02, g02, x02, renorm, prenorm, prenorm_bf16, overwrite_quirk)
        _add_renorm(w1, c1, shadow1, n1, g1, x1, renorm, prenorm, prenorm_bf16, overwrite_quirk)

    res = [o]
    if return_state:
        a02, a1 = weights()
        res += [a02[:, :H].clone(memory_format=torch.contiguous_format), a1.clone(),
                a02[:, H:].clone(memory_format=torch.contiguous_format)]
    if return_momentum:
        res += [m02[:, :H].clone(memory_format=torch.contiguous_format), m1.clone(),
                m02[:, H:].clone(memory_format=torch.contiguous_format)]
    return res[0] if len(res) == 1 else tuple(res)
