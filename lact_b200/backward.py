"""Training backward of the chunk recurrence, chunk by chunk in reverse.

Host orchestration in Python; every contraction runs on the tcgen05 GEMM engine
(`lact_bmm2_bf16`) and every pointwise stage in a CUDA kernel of the library.  The structure
follows the reference's hand-written backward of its two fused autograd Functions
(lact_llm/lact_model/lact_triton_kernels/lact_swiglu_ffn.py:46-76 and lact_fw_grad.py:61-156) and
autograd through the eager momentum / renormalisation lines (ttt_operation.py:170-200).
Like the reference's, the backward recomputes pre-activations in bf16 and returns bf16 gradients
for activations, fp32 for learning rates, momentum and fast weights.

Supported: post-norm and pre-norm recurrences (renorm none / eps outside / eps inside), the
bidirectional overwrite (w <- renorm(NS(dw) + dw)), momentum, any step program, Muon on or off
(Newton-Schulz is recomputed in the backward; its roundings are treated as identities).  Pre-norm
keeps no per-update copy of the un-normalised master weights: they are rebuilt by one forward sweep
over the saved gradients before the reverse sweep.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib as L
from . import program as P

BF16 = torch.bfloat16
_status: Dict[tuple, torch.Tensor] = {}


def _status_word(dev: torch.device) -> torch.Tensor:
    """Device status word of the backward kernels, one per (device, stream)."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), L.stream_ptr())
    if key not in _status:
        _status[key] = torch.zeros(64, dtype=torch.int32, device=dev)
    return _status[key]


def reset_status(dev: torch.device) -> None:
    """Clears the word (stream-ordered): kernels return early while it is non-zero, so a sweep must
    not inherit the failure of an earlier one."""
    _status_word(dev).zero_()


def post_status(dev: torch.device) -> None:
    """After a sweep has been enqueued: its status word travels to the host without waiting for the device and is
    examined at a later library call or in `synchronize_and_check` (see `_lib._StatusRing`)."""
    L.mark_pending(_status_word(dev).view(torch.uint8))


def check_status(dev: torch.device) -> None:
    """Raises if a bounded wait ran out during the sweep; the word is cleared first, so the next
    backward call starts clean."""
    word = _status_word(dev)
    st = int(word[0].item())
    if st != 0:
        word.zero_()
        raise L.LactError(f"device status {st} during backward")


def _strided(t):
    """A [batch, rows, cols] bf16 tensor as (tensor, row stride, batch stride) for the strided GEMM entry; views
    whose innermost axis is contiguous and whose strides / base keep 16-byte alignment pass through uncopied."""
    if t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16 or t.stride(1) < t.shape[2]:
        t = t.contiguous()
    return t, t.stride(1), t.stride(0)


def _desc(a, b, a_mn=False, b_mn=False, a1=None, b1=None, a1_mn=False, b1_mn=False, out=None,
          out_dtype=torch.float32, accumulate=False):
    """(lact_bmm_desc, output tensor, tensors to keep alive) for c[batch, M, N] (+)= a b^T (+ a1 b1^T)."""
    a, a_ld, a_bs = _strided(a)
    b, b_ld, b_bs = _strided(b)
    batch = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mn else (a.shape[1], a.shape[2])
    N = b.shape[2] if b_mn else b.shape[1]
    if out is None:
        out = torch.empty(batch, M, N, dtype=out_dtype, device=a.device)
    assert out.stride(2) == 1 and out.shape == (batch, M, N)
    a1_ld = a1_bs = b1_ld = b1_bs = 0
    if a1 is not None:
        a1, a1_ld, a1_bs = _strided(a1)
        b1, b1_ld, b1_bs = _strided(b1)
    d = L.BmmDesc(a.data_ptr(), b.data_ptr(), a1.data_ptr() if a1 is not None else None,
                  b1.data_ptr() if b1 is not None else None, out.data_ptr(), a_ld, a_bs, b_ld, b_bs, a1_ld, a1_bs,
                  b1_ld, b1_bs, out.stride(1), out.stride(0), batch, M, N, K, int(a_mn), int(b_mn), int(a1_mn),
                  int(b1_mn), L.dtype_code(out), int(accumulate))
    return d, out, (a, b, a1, b1)


def gemm(a, b, **kw):
    """c[batch, M, N] (+)= a b^T (+ a1 b1^T).  Operands bf16, [batch, rows, K] or (``*_mn``) [batch, K, rows];
    operands and `out` may be views into larger tensors (token ranges).  Keywords: a_mn, b_mn, a1, b1, a1_mn, b1_mn,
    out, out_dtype (fp32), accumulate."""
    d, out, _keep = _desc(a, b, **kw)
    rc = L.lib().lact_bmm_group_bf16(C.byref(d), 1, _status_word(out.device).data_ptr(), L.stream_ptr())
    L.check(rc, "lact_bmm_group_bf16")
    return out


def gemm_pair(spec0, spec1):
    """Two independent products (each spec = (a, b, keywords of `gemm`)) in one launch; returns their outputs."""
    d0, out0, _k0 = _desc(spec0[0], spec0[1], **spec0[2])
    d1, out1, _k1 = _desc(spec1[0], spec1[1], **spec1[2])
    pair = (L.BmmDesc * 2)(d0, d1)
    rc = L.lib().lact_bmm_group_bf16(pair, 2, _status_word(out0.device).data_ptr(), L.stream_ptr())
    L.check(rc, "lact_bmm_group_bf16")
    return out0, out1


def _vecptr(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


def _tok_strides(t):
    """A [B, n, D] bf16 activation view as (tensor, token stride, batch stride) for entry points that take strides."""
    if t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16 or t.stride(1) < t.shape[2]:
        t = t.contiguous()
    return t, t.stride(1), t.stride(0)


def apply_backward(w02b, w1b, q, dO, dW02, dW1, dq_out=None):
    """Backward of o = w1 (silu(w0 q) * (w2 q)) on one token range.  Accumulates the weight gradients
    (fp32) into dW02 / dW1 and returns dq (bf16; written into the view `dq_out` if given).
    lact_swiglu_ffn.py:46-76.  Three launches: the pre-activations y0, y2 = q w0^T, q w2^T and dh = dO w1 with the
    pointwise stage in their epilogue (the fast-weight gradient's own kernel with unit learning rates), both weight
    gradients, dq."""
    B, n, D = q.shape
    H = w1b.shape[2]
    dy02 = torch.empty(B, n, 2 * H, dtype=BF16, device=q.device)
    hid = torch.empty(B, n, H, dtype=BF16, device=q.device)
    qs, q_ts, q_bs = _tok_strides(q)
    ds, d_ts, d_bs = _tok_strides(dO)
    L.check(L.lib().lact_fw_grad_pointwise(w02b.data_ptr(), w1b.data_ptr(), qs.data_ptr(), q_ts, q_bs, ds.data_ptr(), d_ts,
                                           d_bs, None, None, None, L.LACT_F32, 0, 1.0, dy02.data_ptr(), hid.data_ptr(),
                                           B, n, D, H, _status_word(q.device).data_ptr(), L.stream_ptr()),
            "lact_fw_grad_pointwise")
    gemm_pair((dy02, q, dict(a_mn=True, b_mn=True, out=dW02, accumulate=True)),     # [2H, D] += dy02^T q
              (dO, hid, dict(a_mn=True, b_mn=True, out=dW1, accumulate=True)))      # [D, H]  += dO^T hidden
    return gemm(dy02, w02b, b_mn=True, out=dq_out, out_dtype=BF16)                  # dq = dy02 w02


def fw_grad_backward(w02b, w1b, k, v, lr0, lr1, lr2, w_scale, gG02, gG1, dW02, dW1, dk_out=None, dv_out=None,
                     g02b=None, g1b=None):
    """Backward of the lr-weighted fast-weight gradient on one token range, given the gradients gG02
    ([B,2H,D]) / gG1 ([B,D,H]) of its outputs.  Accumulates into dW02 / dW1; returns
    (dk, dv [bf16; written into the views `dk_out` / `dv_out` if given], dlr0, dlr1, dlr2 [fp32, B x n]).
    lact_fw_grad.py:61-156.  Products that share a shape class run two per launch."""
    B, n, D = k.shape
    H = w1b.shape[2]
    if g02b is None:
        g02b, g1b = gG02.to(BF16), gG1.to(BF16)
    bf = dict(out_dtype=BF16)
    y02, g_dy02 = gemm_pair((k, w02b, bf), (k, g02b, bf))                                  # [B, n, 2H] each
    dh, g_hid = gemm_pair((v, w1b, dict(b_mn=True, out_dtype=BF16)), (v, g1b, dict(b_mn=True, out_dtype=BF16)))
    g_y02, dy02l = torch.empty_like(y02), torch.empty_like(y02)
    g_dh, hidl = torch.empty_like(dh), torch.empty_like(dh)
    glr = [torch.empty(B, n, dtype=torch.float32, device=k.device) for _ in range(3)]
    lr0, lr1, lr2 = lr0.contiguous(), lr1.contiguous(), lr2.contiguous()
    L.check(L.lib().lact_fw_grad_bwd_pointwise(
        y02.data_ptr(), dh.data_ptr(), g_dy02.data_ptr(), g_hid.data_ptr(), lr0.data_ptr(), lr1.data_ptr(),
        lr2.data_ptr(), L.dtype_code(lr0), float(w_scale), g_y02.data_ptr(), g_dh.data_ptr(), dy02l.data_ptr(),
        hidl.data_ptr(), glr[0].data_ptr(), glr[1].data_ptr(), glr[2].data_ptr(), B * n, H, L.stream_ptr()),
        "lact_fw_grad_bwd_pointwise")
    dk, dv = gemm_pair((g_y02, w02b, dict(b_mn=True, a1=dy02l, b1=g02b, b1_mn=True, out=dk_out, out_dtype=BF16)),
                       (g_dh, w1b, dict(a1=hidl, b1=g1b, out=dv_out, out_dtype=BF16)))
    gemm_pair((g_y02, k, dict(a_mn=True, b_mn=True, out=dW02, accumulate=True)),
              (v, g_dh, dict(a_mn=True, b_mn=True, out=dW1, accumulate=True)))
    return dk, dv, glr[0], glr[1], glr[2]


def renorm_backward(base, upd, n0, dy, dn0, mode, want_bf16=False):
    """dw for y = renorm(base + upd); adds the n0 gradient into dn0.  Rows = all leading dims.  With `want_bf16`
    returns (dw, bf16 copy of dw)."""
    C_ = base.shape[-1]
    rows = base.numel() // C_
    dw = torch.empty_like(base)
    dwb = torch.empty_like(base, dtype=BF16) if want_bf16 else None
    upd = upd.contiguous()
    L.check(L.lib().lact_renorm_bwd(base.data_ptr(), upd.data_ptr(), L.dtype_code(upd), n0.data_ptr(), dy.data_ptr(),
                                    dw.data_ptr(), _vecptr(dwb), _vecptr(dn0), rows, C_, int(mode), L.stream_ptr()),
            "lact_renorm_bwd")
    return (dw, dwb) if want_bf16 else dw


NS_TUNED5 = ((4.0848, -6.8946, 2.9270), (3.9505, -6.3029, 2.6377), (3.7418, -5.5913, 2.3037),
             (2.8769, -3.1427, 1.2046), (2.8366, -3.0525, 1.2012))
NS_CONST = (3.4445, -4.7750, 2.0315)


def ns_forward_saved(G, steps, const_coeffs, gram_right):
    """Recomputes the Newton-Schulz iteration on G [nmat, R, C] keeping every iterate
    (`lact_ns_trace_fwd`: the forward kernels' own arithmetic, iterates in a trace buffer).
    Returns a dict used by `ns_backward` and the result U in G's orientation (bf16)."""
    G = G.contiguous()
    nmat, R, Cc = G.shape
    if G.dtype not in (torch.float32, BF16):
        G = G.float()
    if int(steps) == 0:   # no iteration (lact_nvs/lact_ttt.py with muon_update_steps = 0): the normalisation alone
        from . import ops
        U = ops.zeropower_via_newtonschulz5(G, 0)
        return dict(trace=None, shape=(nmat, R, Cc), steps=0, cc=1, gr=int(bool(gram_right)), G=G), U
    need = C.c_size_t(0)
    L.check(L.lib().lact_ns_trace_bytes(nmat, R, Cc, int(steps), C.byref(need)), "lact_ns_trace_bytes")
    trace = torch.empty(need.value, dtype=torch.uint8, device=G.device)
    U = torch.empty(nmat, R, Cc, dtype=BF16, device=G.device)
    with torch.cuda.device(G.device):
        L.check(L.lib().lact_ns_trace_fwd(G.data_ptr(), L.dtype_code(G), U.data_ptr(), nmat, R, Cc, int(steps),
                                          int(bool(const_coeffs)), int(bool(gram_right)), trace.data_ptr(), trace.numel(),
                                          _status_word(G.device).data_ptr(), L.stream_ptr()), "lact_ns_trace_fwd")
    return dict(trace=trace, shape=(nmat, R, Cc), steps=int(steps), cc=int(bool(const_coeffs)), gr=int(bool(gram_right)),
                G=G), U


def ns_backward(saved, dU):
    """Gradient w.r.t. G of U = NS(G) given dU (fp32, G's orientation): `lact_ns_trace_bwd` walks
    the saved iterates backwards (three two-product contractions per iteration, roundings treated
    as identities, bf16 operands as in the reference's autograd), then the Frobenius
    normalisation X0 = bf16(G) / (||G|| + 1e-7) is differentiated here."""
    nmat, R, Cc = saved["shape"]
    du = (dU if dU.dtype == BF16 else dU.to(BF16)).contiguous()
    dX0 = torch.empty(nmat, R, Cc, dtype=torch.float32, device=du.device)
    trace = saved["trace"]
    if saved["steps"] == 0:
        dX0.copy_(du)
    with torch.cuda.device(du.device):
        if saved["steps"] > 0:
            L.check(L.lib().lact_ns_trace_bwd(du.data_ptr(), dX0.data_ptr(), nmat, R, Cc, saved["steps"], saved["cc"],
                                              saved["gr"], trace.data_ptr(), trace.numel(),
                                              _status_word(du.device).data_ptr(), L.stream_ptr()), "lact_ns_trace_bwd")
    # dX0 / den - bf16(G) <dX0, bf16(G)> / (den^2 ||bf16(G)||), in place in dX0
    G = saved["G"]
    G = G if (G.dtype == torch.float32 and G.is_contiguous()) else G.float().contiguous()
    part = torch.empty(nmat * 2 * L.lib().lact_momentum_bwd_slices(), dtype=torch.float32, device=du.device)
    L.check(L.lib().lact_ns_norm_bwd(G.data_ptr(), dX0.data_ptr(), part.data_ptr(), nmat, R * Cc, L.stream_ptr()),
            "lact_ns_norm_bwd")
    return dX0


def ns_backward_groups(saved, dUs):
    """`ns_backward` for one or two groups of matrices at once: all iterations of all groups in one cooperative
    launch (`lact_ns_trace_bwd_fused`) when an instantiation covers the shapes, else one group after the other."""
    same = all(sv["steps"] == saved[0]["steps"] and sv["cc"] == saved[0]["cc"] and sv["gr"] == saved[0]["gr"]
               for sv in saved)
    if same and 1 <= saved[0]["steps"] <= 5 and len(saved) <= 2:
        dev = dUs[0].device
        slices = L.lib().lact_momentum_bwd_slices()
        groups = (L.NsBwdGroup * len(saved))()
        keep, outs = [], []
        for i, (sv, dU) in enumerate(zip(saved, dUs)):
            nmat, R, Cc = sv["shape"]
            du = (dU if dU.dtype == BF16 else dU.to(BF16)).contiguous()
            G = sv["G"]
            G = G if (G.dtype == torch.float32 and G.is_contiguous()) else G.float().contiguous()
            dg = torch.empty(nmat, R, Cc, dtype=torch.float32, device=dev)
            part = torch.empty(nmat * 2 * slices, dtype=torch.float32, device=dev)
            keep += [du, G, part]
            outs.append(dg)
            groups[i] = L.NsBwdGroup(du.data_ptr(), G.data_ptr(), dg.data_ptr(), sv["trace"].data_ptr(),
                                     sv["trace"].numel(), part.data_ptr(), nmat, R, Cc)
        with torch.cuda.device(dev):
            rc = L.lib().lact_ns_trace_bwd_fused(groups, len(saved), saved[0]["steps"], saved[0]["cc"], saved[0]["gr"],
                                                 _status_word(dev).data_ptr(), L.stream_ptr())
        if rc == 0:
            return outs
        if rc != L.ERR_CONFIG:
            L.check(rc, "lact_ns_trace_bwd_fused")
    return [ns_backward(sv, dU) for sv, dU in zip(saved, dUs)]


def scan_forward_saving(opts, steps, w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum):
    """Forward of the recurrence that also records, per update, the weights it computed with and
    its gradient after momentum (what `scan_backward` needs).  Returns (o, wf0, wf1, wf2, dump)."""
    from . import ops
    if opts.get("prenorm") and opts.get("overwrite_quirk"):
        raise NotImplementedError("no reference recurrence combines pre-norm with the bidirectional overwrite")
    n_upd = sum(1 for s in steps if s[0] == P.UPDATE)
    B, Ltok, D = k.shape
    H = w0.shape[1]
    per = 2 * (B * 2 * H * D + B * D * H)
    dump = torch.empty(max(n_upd, 1), per, dtype=torch.float32, device=q.device)
    # with Muon the forward's own Newton-Schulz iterates are kept too (no recomputation in the backward)
    stride, _ = ops.ns_trace_layout(B, Ltok, D, H, opts) if q.dtype == BF16 else (0, 0)
    ns_dump = torch.empty(max(n_upd, 1) * stride if stride else 1, dtype=torch.uint8, device=q.device)
    with torch.no_grad():
        res = ops.scan_eager(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, momentum=momentum, return_state=True,
                             _state_dump=dump, _ns_trace=ns_dump if stride else None,
                             **{k_: v_ for k_, v_ in opts.items() if k_ not in ("return_state", "_detach_norms")})
    o, wf0, wf1, wf2 = res[:4]
    return o, wf0, wf1, wf2, dump, ns_dump


def ns_saved_from_trace(trace: torch.Tensor, G: torch.Tensor, steps, const_coeffs, gram_right):
    """The `saved` record `ns_backward` expects, built from a trace the training forward kept (no recomputation),
    and the iteration's result U (a bf16 view into the trace)."""
    nmat, R, Cc = G.shape
    off = C.c_size_t(0)
    L.check(L.lib().lact_ns_trace_result_offset(nmat, R, Cc, int(steps), C.byref(off)), "lact_ns_trace_result_offset")
    U = trace[off.value:off.value + nmat * R * Cc * 2].view(BF16).view(nmat, R, Cc)
    return dict(trace=trace, shape=(nmat, R, Cc), steps=int(steps), cc=int(bool(const_coeffs)), gr=int(bool(gram_right)),
                G=G), U


def scan_backward(opts, steps, w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum, dump, wf0, wf1, wf2, dO, gwf=None,
                  ns_dump=None):
    """Reverse sweep over the step program.  `momentum` may be None.  `gwf` = optional cotangents
    (g_w0, g_w1, g_w2; any may be None) of the final fast weights the forward returned: they seed
    the weight gradient the sweep starts from (in the reference the returned weights carry autograd
    history, e.g. lact_nvs/lact_ttt.py:147).  Returns the gradients of
    (w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum) (the last one None without momentum)."""
    has_momentum = momentum is not None
    n_upd = sum(1 for s_ in steps if s_[0] == P.UPDATE)
    reset_status(q.device)
    dev = q.device
    B, Ltok, D = k.shape
    H = w0.shape[1]
    n02, n1 = B * 2 * H * D, B * D * H
    mode = int(opts.get("renorm", L.RENORM_EPS_OUTSIDE))
    w_scale = float(opts.get("w_scale", 1.0))
    f32 = torch.float32
    vec = lambda t: (t[..., 0] if t.dim() == 3 else t).contiguous()
    lr0v, lr1v, lr2v = vec(lr0), vec(lr1), vec(lr2)
    momv = vec(momentum).float() if has_momentum else None
    W0_02 = torch.cat([w0, w2], dim=1).float().contiguous()
    W0_1 = w1.float().contiguous()
    n0_02 = W0_02.norm(dim=2).contiguous()
    n0_1 = W0_1.norm(dim=2).contiguous()

    def weights(cnt):
        """fp32 (W02, W1) in force after `cnt` updates."""
        if cnt == 0:
            return W0_02, W0_1
        if cnt < n_upd:
            return dump[cnt, :n02].view(B, 2 * H, D), dump[cnt, n02:n02 + n1].view(B, D, H)
        return torch.cat([wf0, wf2], dim=1).contiguous(), wf1.contiguous()

    def grad_state(u):
        """fp32 gradient after momentum of update u (= momentum state after it)."""
        base = n02 + n1
        return dump[u, base:base + n02].view(B, 2 * H, D), dump[u, base + n02:base + n02 + n1].view(B, D, H)

    ns_stride = ns_off1 = 0
    if ns_dump is not None:
        from . import ops as _ops
        ns_stride, ns_off1 = _ops.ns_trace_layout(B, Ltok, D, H, opts)
        if ns_stride == 0:
            ns_dump = None
    prenorm, muon = bool(opts.get("prenorm")), bool(opts.get("use_muon"))
    overwrite = bool(opts.get("overwrite_quirk")) and muon
    nst, cc, gr = int(opts.get("ns_steps", 5)), bool(opts.get("ns_const_coeffs")), bool(opts.get("ns_gram_right"))

    # pre-norm: master weights before each update, Wm_0 = W_0, Wm_{u+1} = Wm_u + U_u
    masters = None
    if prenorm:
        from . import ops

        def fast_ns(g):
            st = nst if cc else None
            if gr:
                return ops.zeropower_via_newtonschulz5(g.transpose(1, 2).contiguous(), st).transpose(1, 2)
            return ops.zeropower_via_newtonschulz5(g, st)

        def kept_result(u, group):
            """Newton-Schulz result of update u as the forward kept it (bf16 view into its trace)."""
            tr = ns_dump[u * ns_stride:(u + 1) * ns_stride]
            tr = tr[:ns_off1] if group == 0 else tr[ns_off1:]
            nmat, R, Cc = ((B, 2 * H, D) if opts.get("ns_concat") else (2 * B, H, D)) if group == 0 else (B, D, H)
            off = C.c_size_t(0)
            L.check(L.lib().lact_ns_trace_result_offset(nmat, R, Cc, nst, C.byref(off)), "lact_ns_trace_result_offset")
            x = tr[off.value:off.value + nmat * R * Cc * 2].view(BF16)
            return x.view(B, 2 * H, D) if group == 0 else x.view(B, D, H)

        masters = [(W0_02, W0_1)]
        for u in range(n_upd - 1):
            g02, g1 = grad_state(u)
            if muon and ns_dump is not None:
                g02, g1 = kept_result(u, 0), kept_result(u, 1)
            elif muon:
                g02 = fast_ns(g02) if opts.get("ns_concat") else torch.cat(
                    [fast_ns(g02[:, :H]), fast_ns(g02[:, H:])], dim=1)
                g1 = fast_ns(g1)
            masters.append((masters[-1][0] + g02.float(), masters[-1][1] + g1.float()))

    dW02 = torch.zeros(B, 2 * H, D, dtype=f32, device=dev)
    dW1 = torch.zeros(B, D, H, dtype=f32, device=dev)
    if gwf is not None:  # cotangents of the returned final weights (the compute copy after the last update)
        if gwf[0] is not None:
            dW02[:, :H] = gwf[0]
        if gwf[2] is not None:
            dW02[:, H:] = gwf[2]
        if gwf[1] is not None:
            dW1.copy_(gwf[1])
    dWm02 = dWm1 = None  # pre-norm: gradient w.r.t. the master weights after the current update
    dM02 = dM1 = None
    dn02 = torch.zeros(B, 2 * H, dtype=f32, device=dev)
    dn1 = torch.zeros(B, D, dtype=f32, device=dev)
    # every token range is written in place by the first step that produces a gradient for it: only the gaps no
    # step covers are zero-filled
    def gaps(kind_):
        out_, end_ = [], 0
        for s_, e_ in sorted((st[1], st[2]) for st in steps if st[0] == kind_ and st[2] > st[1]):
            if s_ > end_:
                out_.append((end_, s_))
            end_ = max(end_, e_)
        if end_ < Ltok:
            out_.append((end_, Ltok))
        return out_
    dq, dk, dv = torch.empty_like(q, dtype=BF16), torch.empty_like(k, dtype=BF16), torch.empty_like(v, dtype=BF16)
    for a_, b_ in gaps(P.APPLY):
        dq[:, a_:b_].zero_()
    for a_, b_ in gaps(P.UPDATE):
        dk[:, a_:b_].zero_()
        dv[:, a_:b_].zero_()
    dlr = [torch.zeros(B, Ltok, dtype=f32, device=dev) for _ in range(3)]
    dmom = torch.zeros(B, Ltok, dtype=f32, device=dev) if has_momentum else None
    dO = dO.to(BF16)

    # learning rates of the update steps as contiguous [B, n] blocks: one copy per sweep when the steps tile a token
    # range back to back with one length (the usual chunking), else one small copy per step
    upd_steps = [(st[1], st[2]) for st in steps if st[0] == P.UPDATE and st[2] > st[1]]
    lr_blocks = None
    if upd_steps:
        n_ = upd_steps[0][1] - upd_steps[0][0]
        if all(e_ - s_ == n_ for s_, e_ in upd_steps) and all(upd_steps[i + 1][0] == upd_steps[i][1]
                                                              for i in range(len(upd_steps) - 1)):
            s0_, e1_ = upd_steps[0][0], upd_steps[-1][1]
            blk = lambda t: t[:, s0_:e1_].reshape(B, len(upd_steps), n_).transpose(0, 1).contiguous()
            lr_blocks = (s0_, n_, blk(lr0v), blk(lr1v), blk(lr2v))

    def lr_slices(s_, e_):
        if lr_blocks is not None:
            i_ = (s_ - lr_blocks[0]) // lr_blocks[1]
            return lr_blocks[2][i_], lr_blocks[3][i_], lr_blocks[4][i_]
        return lr0v[:, s_:e_], lr1v[:, s_:e_], lr2v[:, s_:e_]

    cnt = n_upd
    shadows = {}
    q_done, kv_done = [], []  # token ranges whose dq / dk, dv have been written

    def fresh(done, s_, e_):
        """True (and records the range) if no earlier step wrote a gradient for tokens [s_, e_)."""
        ok = all(e_ <= a_ or s_ >= b_ for a_, b_ in done)
        done.append((s_, e_))
        return ok

    def shadow(c_):
        if c_ not in shadows:
            shadows.clear()
            a, b = weights(c_)
            shadows[c_] = (a.to(BF16).contiguous(), b.to(BF16).contiguous())
        return shadows[c_]

    for kind, s, e, o_s in reversed(steps):
        if e <= s:
            continue
        if kind == P.APPLY:
            w02b, w1b = shadow(cnt)
            if fresh(q_done, s, e):   # first gradient for these tokens: the product writes it in place
                apply_backward(w02b, w1b, q[:, s:e], dO[:, o_s:o_s + (e - s)], dW02, dW1, dq_out=dq[:, s:e])
            else:
                dq[:, s:e] += apply_backward(w02b, w1b, q[:, s:e], dO[:, o_s:o_s + (e - s)], dW02, dW1)
            continue
        u = cnt - 1
        Wp02, Wp1 = weights(u)
        G02, G1 = grad_state(u)
        # update applied to the weights: the gradient itself, or its Newton-Schulz image (recomputed)
        U02, U1, sv02, sv1 = G02.contiguous(), G1.contiguous(), None, None
        if muon:
            g02m = G02.contiguous() if opts.get("ns_concat") else G02.contiguous().view(2 * B, H, D)
            if ns_dump is not None:
                tr = ns_dump[u * ns_stride:(u + 1) * ns_stride]
                sv02, U02 = ns_saved_from_trace(tr[:ns_off1], g02m, nst, cc, gr)
                sv1, U1 = ns_saved_from_trace(tr[ns_off1:], G1.contiguous(), nst, cc, gr)
            else:
                sv02, U02 = ns_forward_saved(g02m, nst, cc, gr)
                sv1, U1 = ns_forward_saved(G1.contiguous(), nst, cc, gr)
            U02 = U02.view(B, 2 * H, D)
        # renorm backward: dWn is the gradient w.r.t. (base + update); base is W_u, the master
        # copy (pre-norm), or the gradient itself (bidirectional overwrite)
        if prenorm:
            b02, b1 = masters[u]
        elif overwrite:
            b02, b1 = G02, G1
        else:
            b02, b1 = Wp02, Wp1
        carry_in = prenorm and dWm02 is not None
        want_b = sv02 is not None and not carry_in
        r02 = renorm_backward(b02.contiguous(), U02, n0_02, dW02, dn02, mode, want_bf16=want_b)
        r1 = renorm_backward(b1.contiguous(), U1, n0_1, dW1, dn1, mode, want_bf16=want_b)
        (dWn02, dWn02b), (dWn1, dWn1b) = (r02, r1) if want_b else ((r02, None), (r1, None))
        if carry_in:
            dWn02 += dWm02
            dWn1 += dWm1
        if sv02 is not None:
            dG02, dG1 = ns_backward_groups([sv02, sv1], [(dWn02b if dWn02b is not None else dWn02).view(sv02["shape"]),
                                                         dWn1b if dWn1b is not None else dWn1])
            dG02 = dG02.view(B, 2 * H, D)
            if overwrite:
                dG02 += dWn02
                dG1 += dWn1
        else:
            dG02, dG1 = dWn02.clone(), dWn1.clone()
        if prenorm:        # the weights update u computed with receive gradient only from its own steps
            dWm02, dWm1 = dWn02, dWn1
            dW02, dW1 = torch.zeros_like(dWn02), torch.zeros_like(dWn1)
        elif overwrite:    # the previous weights were overwritten: no direct path
            dW02, dW1 = torch.zeros_like(dWn02), torch.zeros_like(dWn1)
        else:
            dW02, dW1 = dWn02, dWn1
        # momentum step (one kernel): dG += what arrives from the next update's momentum state, dbeta, the share
        # that goes on to the previous update, and the bf16 copies the contractions below read
        g02b, g1b = torch.empty_like(dG02, dtype=BF16), torch.empty_like(dG1, dtype=BF16)
        beta = dbeta = None
        mp02 = mp1 = None
        if has_momentum:
            beta = momv[:, s:e].mean(dim=1).contiguous()  # [B]
            if u > 0:
                mp02, mp1 = grad_state(u - 1)
                dbeta = torch.empty(B, L.lib().lact_momentum_bwd_slices(), dtype=f32, device=dev)
            if dM02 is None:
                dM02, dM1, add_carry = torch.empty_like(dG02), torch.empty_like(dG1), 0
            else:
                add_carry = 1
        L.check(L.lib().lact_momentum_bwd(dG02.data_ptr(), dG1.data_ptr(), _vecptr(dM02 if has_momentum else None),
                                          _vecptr(dM1 if has_momentum else None), _vecptr(mp02), _vecptr(mp1),
                                          g02b.data_ptr(), g1b.data_ptr(), _vecptr(beta), _vecptr(dbeta), B, 2 * H * D,
                                          D * H, add_carry if has_momentum else 0, L.stream_ptr()), "lact_momentum_bwd")
        if dbeta is not None:
            dmom[:, s:e] += (dbeta.sum(dim=1) / float(e - s)).unsqueeze(1)
        w02b, w1b = shadow(u)
        l0_, l1_, l2_ = lr_slices(s, e)
        if fresh(kv_done, s, e):
            _, _, g0, g1, g2 = fw_grad_backward(w02b, w1b, k[:, s:e], v[:, s:e], l0_, l1_, l2_, w_scale, dG02, dG1,
                                                dW02, dW1, dk_out=dk[:, s:e], dv_out=dv[:, s:e], g02b=g02b, g1b=g1b)
        else:
            gk, gv, g0, g1, g2 = fw_grad_backward(w02b, w1b, k[:, s:e], v[:, s:e], l0_, l1_, l2_, w_scale, dG02, dG1,
                                                  dW02, dW1, g02b=g02b, g1b=g1b)
            dk[:, s:e] += gk
            dv[:, s:e] += gv
        dlr[0][:, s:e] += g0
        dlr[1][:, s:e] += g1
        dlr[2][:, s:e] += g2
        cnt = u
    post_status(dev)
    if dWm02 is not None:  # W_0 is both the first master and the first compute copy
        dW02, dW1 = dW02 + dWm02, dW1 + dWm1
    # the target row norms are functions of the initial weights (not detached in the LLM / AR paths)
    if not opts.get("_detach_norms", False):
        dW02 = dW02 + dn02.unsqueeze(-1) * W0_02 / n0_02.clamp_min(1e-30).unsqueeze(-1)
        dW1 = dW1 + dn1.unsqueeze(-1) * W0_1 / n0_1.clamp_min(1e-30).unsqueeze(-1)
    dw0, dw2 = dW02[:, :H].to(w0.dtype), dW02[:, H:].to(w2.dtype)
    shape = lambda g, ref: g.view(ref.shape).to(ref.dtype) if ref.dim() == 3 else g.to(ref.dtype)
    grads = (dw0, dW1.to(w1.dtype), dw2, dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype),
             shape(dlr[0].unsqueeze(-1) if lr0.dim() == 3 else dlr[0], lr0),
             shape(dlr[1].unsqueeze(-1) if lr1.dim() == 3 else dlr[1], lr1),
             shape(dlr[2].unsqueeze(-1) if lr2.dim() == 3 else dlr[2], lr2),
             shape(dmom.unsqueeze(-1) if momentum.dim() == 3 else dmom, momentum) if has_momentum else None)
    return grads
