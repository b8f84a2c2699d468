"""CPU oracle for the LaCT large-chunk fast-weight TTT step.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this module; it is
used by the tests, by the smoke check and by the CPU-baseline leg of the benchmark as the
checker / timed CPU baseline, never as the thing shipped.

It restates, with plain PyTorch CPU tensor ops, the algorithm of the reference repository
a1600012888/LaCT for this path.  Every public function names the reference file:line it
follows.  Two numerics policies exist:

* ``policy="ref"``  - the arithmetic of the reference's *unfused* PyTorch functions, dtype for
  dtype (fp32 inputs run in fp32; ``autocast=True`` emulates ``torch.autocast(bfloat16)`` by
  casting both bmm operands to bf16).  With fp32 inputs it is bit-identical on CPU to the
  reference functions; the committed fixtures under ``tests/golden`` (made by importing the
  reference, see ``tests/golden/make_golden.py``) pin that.
* ``policy="fused"`` - the rounding model of the reference's fused (Triton) path, which is
  also the rounding model of the CUDA kernels: bf16 operands, fp32 accumulators, fp32
  epilogue math, one rounding to bf16 when a tile is stored, bf16 batched-GEMM outputs,
  fp32 momentum / renormalisation, Newton-Schulz in bf16.

Parity status: PINNED against outputs of the reference itself (fixtures generated in the build
container by running the reference functions on CPU in eager mode).  The reference ships no
golden vectors or tests of its own for this path.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

BF16 = torch.bfloat16

# Newton-Schulz coefficient triples.
# Tuned five-step table: lact_llm/lact_model/ttt_operation.py:49-55 (same in
# ttt_operation_fused_kernel.py:46-52, minimal_implementations/bidirectional_lact_layer.py:53-59).
NS_TUNED5 = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)
# Constant triple: lact_nvs/lact_ttt.py:50, lact_ar_video/minVid/models/blocks/functions.py:56.
NS_CONST = (3.4445, -4.7750, 2.0315)


# ----------------------------------------------------------------------------------------------
# small helpers
# ----------------------------------------------------------------------------------------------
def silu_backprop(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """d/dx of silu applied to dy.  lact_llm/lact_model/ttt_operation.py:5-17."""
    sigma = torch.sigmoid(x)
    return dy * sigma * (1 + x * (1 - sigma))


def newton_schulz(G: torch.Tensor, steps: Optional[int] = None) -> torch.Tensor:
    """Batched Newton-Schulz orthogonalisation in bf16 with the reference's eager rounding points.

    ``steps=None``: tuned 5-triple table, lact_llm/lact_model/ttt_operation.py:30-66.
    ``steps=int`` : constant triple repeated ``steps`` times, lact_nvs/lact_ttt.py:32-67.
    """
    assert G.dim() == 3
    coeffs = NS_TUNED5 if steps is None else (NS_CONST,) * steps
    X = G.bfloat16()
    flip = G.size(1) > G.size(2)
    if flip:
        X = X.transpose(1, 2)
    X = X / (X.norm(dim=(1, 2), keepdim=True) + 1e-7)
    for a, b, c in coeffs:
        A = X @ X.transpose(1, 2)
        B = b * A + c * A @ A
        X = a * X + B @ X
    if flip:
        X = X.transpose(1, 2)
    return X


def newton_schulz_folded(G: torch.Tensor, steps: Optional[int] = None, fold_norm: bool = False) -> torch.Tensor:
    """Rounding model of the CUDA kernels' Newton-Schulz: the same iteration with the residual terms
    folded into the contractions as multiples of the identity by completing the square,
    ``S = A + (b/2c) I``, ``a I + b A + c A A = c S S + (a - b^2/4c) I``, ``X' = P X``; bf16 values,
    fp32 accumulation, one rounding per stored matrix (S, P, X').  The reference's compiled GPU graph
    likewise rounds ``b*A + c*A@A`` and ``a*X + B@X`` once (inductor fuses the elementwise part), so its
    own GPU and eager CPU results differ by the same kind of amount as this model and `newton_schulz`.
    ``fold_norm``: the chunk recurrence also folds the Frobenius normalisation into the first
    iteration: it iterates on bf16(G) itself and multiplies the first Gram matrix by s^2 and the
    first update by s, s = 1 / (||G|| + 1e-7), in fp32 before the rounding.
    """
    assert G.dim() == 3
    coeffs = NS_TUNED5 if steps is None else (NS_CONST,) * steps
    X = G.bfloat16()
    flip = G.size(1) > G.size(2)
    if flip:
        X = X.transpose(1, 2)
    den = X.norm(dim=(1, 2), keepdim=True) + 1e-7
    s = (1.0 / den.float()) if (fold_norm and len(coeffs) > 0) else None
    if s is None:
        X = X / den
    eye = torch.eye(X.size(1), dtype=torch.float32)
    for i, (a, b, c) in enumerate(coeffs):
        Xf = X.float()
        s2, s1 = (s * s, s) if (s is not None and i == 0) else (1.0, 1.0)
        S = ((Xf @ Xf.transpose(1, 2)) * s2 + (b / (2.0 * c)) * eye).to(BF16)
        P = (c * (S.float() @ S.float()) + (a - b * b / (4.0 * c)) * eye).to(BF16)
        X = ((P.float() @ Xf) * s1).to(BF16)
    if flip:
        X = X.transpose(1, 2)
    return X


def newton_schulz_f64(G: torch.Tensor, steps: Optional[int] = None) -> torch.Tensor:
    """The same iteration carried out in float64 on the bf16-rounded input (accuracy yardstick)."""
    coeffs = NS_TUNED5 if steps is None else (NS_CONST,) * steps
    X = G.bfloat16().double()
    flip = G.size(1) > G.size(2)
    if flip:
        X = X.transpose(1, 2)
    X = X / (X.norm(dim=(1, 2), keepdim=True) + 1e-7)
    for a, b, c in coeffs:
        A = X @ X.transpose(1, 2)
        B = b * A + (c * A) @ A
        X = a * X + B @ X
    if flip:
        X = X.transpose(1, 2)
    return X


@dataclasses.dataclass
class Numerics:
    """Numerics policy (see module docstring)."""

    policy: str = "ref"  # "ref" | "fused"
    autocast: bool = False  # ref policy: emulate torch.autocast(bfloat16) around bmm


def _bmm(a: torch.Tensor, b: torch.Tensor, nm: Numerics) -> torch.Tensor:
    if nm.autocast:
        return torch.bmm(a.to(BF16), b.to(BF16))
    return torch.bmm(a, b)


def _f32mm_round(a: torch.Tensor, b: torch.Tensor, out_dtype) -> torch.Tensor:
    """GEMM with fp32 accumulation of (bf16-valued) operands, one rounding at the store."""
    return torch.bmm(a.float(), b.float()).to(out_dtype)


# ----------------------------------------------------------------------------------------------
# apply / fast-weight gradient, LLM layout (w0,w2: [B,H,D], w1: [B,D,H])
# ----------------------------------------------------------------------------------------------
def apply_ref(w0, w1, w2, q, nm: Numerics) -> torch.Tensor:
    """o = w1 (silu(w0 q^T) * (w2 q^T)), returned as [B, l, D].

    lact_llm/lact_model/ttt_operation.py:139-144 (also :203-212).
    """
    qt = q.transpose(1, 2)
    h = _bmm(w2, qt, nm)
    gate = F.silu(_bmm(w0, qt, nm))
    return _bmm(w1, gate * h, nm).transpose(1, 2)


def grads_ref(w0, w1, w2, k, v, lr0, lr1, lr2, nm: Numerics, style: str = "llm", w_scale: float = 1.0):
    """Per-token-lr weighted gradient of -<f(k), v> w.r.t. w0, w1, w2 (to be ADDED to the weights).

    style "llm": lact_llm/lact_model/ttt_operation.py:146-168 (lr-scaled operand cast back with
    type_as);  style "ar": lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:110-138
    (lr * w_scale, no cast).
    """
    kt = k.transpose(1, 2)
    vt = v.transpose(1, 2)
    g = _bmm(w0, kt, nm)
    h = _bmm(w2, kt, nm)
    silu_g = F.silu(g)
    hidden = silu_g * h
    dhidden = _bmm(w1.transpose(1, 2), vt, nm)
    dh2 = dhidden * silu_g
    dg = silu_backprop(dhidden * h, g)
    if style == "llm":
        dw1 = _bmm(vt, (hidden.transpose(1, 2) * lr1).type_as(vt), nm)
        dw0 = _bmm(dg, (k * lr0).type_as(dg), nm)
        dw2 = _bmm(dh2, (k * lr2).type_as(dh2), nm)
    else:
        dw1 = _bmm(vt, hidden.transpose(1, 2) * lr1 * w_scale, nm)
        dw0 = _bmm(dg, k * lr0 * w_scale, nm)
        dw2 = _bmm(dh2, k * lr2 * w_scale, nm)
    return dw0, dw1, dw2


def apply_fused(w0w2_b, w1_b, q) -> torch.Tensor:
    """Fused-path apply: bf16 operands, fp32 SwiGLU epilogue, hidden rounded to bf16, bf16 out.

    lact_llm/lact_model/lact_triton_kernels/lact_swiglu_ffn.py:19-44 with the kernel epilogue of
    triton_swiglu_kernels.py:111-120; formula = reference_swiglu_ffn_fwd (lact_swiglu_ffn.py:104-116).
    """
    H = w0w2_b.shape[1] // 2
    x = q.float().transpose(1, 2)
    y0 = torch.bmm(w0w2_b[:, :H].float(), x)
    y2 = torch.bmm(w0w2_b[:, H:].float(), x)
    hidden = (y2 * (y0 * torch.sigmoid(y0))).to(q.dtype)  # [B,H,l]
    return _f32mm_round(hidden.transpose(1, 2), w1_b.transpose(1, 2), q.dtype)


def grads_fused(w0w2_b, w1_b, k, v, lr0, lr1, lr2, w_scale: float = 1.0):
    """Fused-path gradient (DW0|DW2 [B,2H,D], DW1 [B,D,H]); lr are [B,l].

    lact_llm/lact_model/lact_triton_kernels/lact_fw_grad.py:21-58; epilogue
    triton_swiglu_bwd_with_lr.py:134-194; formula = reference_lact_swiglu_ffn_fast_weight_grads
    (lact_fw_grad.py:268-306).
    """
    H = w0w2_b.shape[1] // 2
    dt = k.dtype
    kt = k.float().transpose(1, 2)
    y0 = torch.bmm(w0w2_b[:, :H].float(), kt)
    y2 = torch.bmm(w0w2_b[:, H:].float(), kt)
    dh = torch.bmm(w1_b.float().transpose(1, 2), v.float().transpose(1, 2))
    sigma = torch.sigmoid(y0)
    swish = sigma * y0
    l0 = (lr0.float() * w_scale).unsqueeze(1)
    l1 = (lr1.float() * w_scale).unsqueeze(1)
    l2 = (lr2.float() * w_scale).unsqueeze(1)
    hidden = (swish * y2 * l1).to(dt)
    dy0 = (sigma * y2 * dh * (1.0 + y0 * (1.0 - sigma)) * l0).to(dt)
    dy2 = (swish * dh * l2).to(dt)
    dy = torch.cat([dy0, dy2], dim=1)
    dw0w2 = _f32mm_round(dy, k, dt)
    dw1 = _f32mm_round(v.transpose(1, 2), hidden.transpose(1, 2), dt)
    return dw0w2, dw1


def l2_norm_add(x, x_add, tgt_scale, eps: float = 1e-5):
    """(x + x_add) * rsqrt(sum((x + x_add)^2) + eps) * scale, eps INSIDE the square root.

    lact_llm/lact_model/lact_triton_kernels/l2norm_triton_kernels.py:430-440 (kernel :60-94).
    """
    y = x.to(torch.float32) + x_add.to(torch.float32)
    rstd = 1 / torch.sqrt(torch.sum(y * y, dim=2, keepdim=True) + eps)
    return y * rstd * tgt_scale.unsqueeze(-1)


def prenorm_update_with_momentum(x, dx, dx_momentum, momentum_mu, tgt_scale, eps: float = 1e-5):
    """m = dx + mu*m; x += m; y = x / sqrt(sum x^2 + eps) * scale (bf16).

    lact_llm/lact_model/lact_triton_kernels/triton_prenorm_update_with_momentum.py:10-38.
    """
    m = dx + dx_momentum * momentum_mu.unsqueeze(-1).unsqueeze(-1)
    x_new = x + m
    denom = torch.sqrt(torch.sum(x_new ** 2, dim=-1, keepdim=True) + eps)
    return x_new, m, (x_new / denom * tgt_scale.unsqueeze(-1)).to(BF16)


def _renorm_outer(w, n0):
    """w / (||w|| + 1e-5) * n0 along dim 2.  lact_llm/lact_model/ttt_operation.py:198-200."""
    return w / (w.norm(dim=2, keepdim=True) + 1e-5) * n0


# ----------------------------------------------------------------------------------------------
# chunk drivers.  Every driver can record the (kind, start, end) steps it executes in `trace`.
# ----------------------------------------------------------------------------------------------
def _rec(trace, kind, s, e, out=None):
    if trace is not None:
        trace.append((kind, int(s), int(e), int(s if out is None else out)))


def block_causal_lact_swiglu(
    w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size=2048, use_muon=False, momentum=None,
    *, prenorm=False, nm: Numerics = Numerics(), trace: Optional[list] = None, states: Optional[list] = None,
):
    """Causal apply-then-update chunk recurrence, unfused arithmetic.

    Post-norm: lact_llm/lact_model/ttt_operation.py:69-214 (identical to
    minimal_implementations/causal_lact_with_sliding_window_attn.py:83-211).
    Pre-norm (``prenorm=True``): lact_llm/lact_model/ttt_operation.py:217-364.
    ``states`` (optional list) receives (w0, w1, w2) after every update, for teacher-forced checks.
    """
    n0, n1, n2 = (w.norm(dim=2, keepdim=True) for w in (w0, w1, w2))
    m0 = m1 = m2 = None
    if momentum is not None:
        m0, m1, m2 = torch.zeros_like(w0), torch.zeros_like(w1), torch.zeros_like(w2)
    w0m, w1m, w2m = w0, w1, w2  # pre-norm master copies
    L = k.shape[1]
    out = torch.zeros_like(v)
    e = 0
    for s in range(0, L - chunk_size, chunk_size):
        e = s + chunk_size
        _rec(trace, "apply", s, e)
        out[:, s:e] = apply_ref(w0, w1, w2, q[:, s:e], nm)
        _rec(trace, "update", s, e)
        dw0, dw1, dw2 = grads_ref(w0, w1, w2, k[:, s:e], v[:, s:e], lr0[:, s:e], lr1[:, s:e], lr2[:, s:e], nm)
        if momentum is not None:
            beta = momentum[:, s:e].mean(dim=1, keepdim=True)
            dw0 = dw0 + m0 * beta
            dw1 = dw1 + m1 * beta
            dw2 = dw2 + m2 * beta
            m0, m1, m2 = dw0, dw1, dw2
        if use_muon:
            dw1 = newton_schulz(dw1)
            dw0 = newton_schulz(dw0)
            dw2 = newton_schulz(dw2)
        if prenorm:
            w1m, w0m, w2m = w1m + dw1, w0m + dw0, w2m + dw2
            w0, w1, w2 = _renorm_outer(w0m, n0), _renorm_outer(w1m, n1), _renorm_outer(w2m, n2)
        else:
            w1, w0, w2 = w1 + dw1, w0 + dw0, w2 + dw2
            w0, w1, w2 = _renorm_outer(w0, n0), _renorm_outer(w1, n1), _renorm_outer(w2, n2)
        if states is not None:
            states.append((w0, w1, w2))
    _rec(trace, "apply", e, L)
    out[:, e:L] = apply_ref(w0, w1, w2, q[:, e:L], nm)
    return out


def block_causal_lact_swiglu_fused(
    w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size=2048, use_muon=False, momentum=None,
    *, prenorm=False, trace: Optional[list] = None, states: Optional[list] = None,
    teacher: Optional[Sequence[Tuple[torch.Tensor, torch.Tensor]]] = None, ns=None,
):
    """Causal apply-then-update recurrence with the fused path's semantics and rounding.
    ``ns``: the Newton-Schulz function (default `newton_schulz`, the reference's eager rounding;
    `newton_schulz_folded` gives the CUDA kernels' rounding).

    Post-norm: lact_llm/lact_model/ttt_operation_fused_kernel.py:66-186; pre-norm: :189-316.
    Differences from the unfused functions that are reproduced here: zero padding to a chunk
    multiple (:112-122), Newton-Schulz on the concatenated [2H, D] matrix (:169-171), renorm
    with eps inside the square root (post-norm, :173-174), bf16 weight shadows (:151-152).
    ``teacher``: optional list of (w0w2, w1) master states to substitute after update i.
    """
    w0w2 = torch.cat([w0, w2], dim=1).contiguous()
    n02 = w0w2.norm(dim=2, keepdim=prenorm)
    n1 = w1.norm(dim=2, keepdim=prenorm)
    w0w2_main, w1_main = w0w2, w1
    if prenorm:
        w0w2, w1 = w0w2.to(BF16), w1.to(BF16)
    m02 = m1 = None
    if momentum is not None:
        m02, m1 = torch.zeros_like(w0w2_main), torch.zeros_like(w1_main)
    L = q.shape[1]
    C = chunk_size
    pad = -L % C
    padf = lambda t: F.pad(t, (0, 0, 0, pad))
    qp, kp, vp = padf(q), padf(k), padf(v)
    l0, l1, l2 = (padf(t)[..., 0] for t in (lr0, lr1, lr2))
    mp = padf(momentum) if momentum is not None else None
    n_chunks = (L + pad + C - 1) // C
    out = torch.zeros_like(qp)
    for ci in range(n_chunks - 1):
        s, e = ci * C, (ci + 1) * C
        w02b, w1b = w0w2.to(BF16), w1.to(BF16)
        _rec(trace, "apply", s, e)
        out[:, s:e] = apply_fused(w02b, w1b, qp[:, s:e])
        _rec(trace, "update", s, e)
        dw02, dw1 = grads_fused(w02b, w1b, kp[:, s:e], vp[:, s:e], l0[:, s:e], l1[:, s:e], l2[:, s:e])
        if momentum is not None:
            beta = mp[:, s:e].mean(dim=1, keepdim=True)
            dw02 = dw02 + m02 * beta
            dw1 = dw1 + m1 * beta
            m02, m1 = dw02, dw1
        if use_muon:
            dw1 = (ns or newton_schulz)(dw1)
            dw02 = (ns or newton_schulz)(dw02)
        if prenorm:
            w0w2_main = w0w2_main + dw02
            w1_main = w1_main + dw1
            w0w2 = (w0w2_main / (w0w2_main.norm(dim=2, keepdim=True) + 1e-5) * n02).to(BF16)
            w1 = (w1_main / (w1_main.norm(dim=2, keepdim=True) + 1e-5) * n1).to(BF16)
        else:
            w0w2 = l2_norm_add(w0w2, dw02, n02, eps=1e-5)
            w1 = l2_norm_add(w1, dw1, n1, eps=1e-5)
        if teacher is not None:
            if prenorm:
                w0w2_main, w1_main = teacher[ci]
                w0w2 = (w0w2_main / (w0w2_main.norm(dim=2, keepdim=True) + 1e-5) * n02).to(BF16)
                w1 = (w1_main / (w1_main.norm(dim=2, keepdim=True) + 1e-5) * n1).to(BF16)
            else:
                w0w2, w1 = teacher[ci]
        if states is not None:
            states.append((w0w2_main, w1_main) if prenorm else (w0w2, w1))
    s = (n_chunks - 1) * C
    _rec(trace, "apply", s, L)
    out[:, s:] = apply_fused(w0w2.to(BF16), w1.to(BF16), qp[:, s:])
    return out[:, :L]


def bidirectional_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, use_muon=True,
                              *, nm: Numerics = Numerics(), trace: Optional[list] = None):
    """One update on all tokens, then apply to all tokens.

    minimal_implementations/bidirectional_lact_layer.py:73-160, INCLUDING its quirk (:139-146):
    with Muon the weights are first overwritten by NS(dw) and the raw dw is then added, i.e.
    w <- renorm(NS(dw) + dw).
    """
    n0, n1, n2 = (w.norm(dim=2, keepdim=True) for w in (w0, w1, w2))
    L = k.shape[1]
    _rec(trace, "update", 0, L)
    dw0, dw1, dw2 = grads_ref(w0, w1, w2, k, v, lr0, lr1, lr2, nm)
    if use_muon:
        w0 = newton_schulz(dw0)
        w1 = newton_schulz(dw1)
        w2 = newton_schulz(dw2)
    w1, w0, w2 = w1 + dw1, w0 + dw0, w2 + dw2
    w0, w1, w2 = _renorm_outer(w0, n0), _renorm_outer(w1, n1), _renorm_outer(w2, n2)
    _rec(trace, "apply", 0, L)
    return apply_ref(w0, w1, w2, q, nm)


def nvs_mini_batch_apply(w0, w1, w2, q, k, v, lr0, lr1, lr2, ttt_ua_order, muon_update_steps=0,
                         *, nm: Numerics = Numerics(), trace: Optional[list] = None):
    """Operator-list driver in the NVS (transposed) layout: w0,w2 [B,D,H], w1 [B,H,D].

    lact_nvs/lact_ttt.py:70-147.  Every update runs Newton-Schulz with the constant triple for
    ``muon_update_steps`` iterations (0 iterations still normalises by the Frobenius norm);
    norms are taken along dim 1; outputs of apply operators are concatenated in list order.
    """
    mm = (lambda a, b: a.to(BF16) @ b.to(BF16)) if nm.autocast else (lambda a, b: a @ b)
    n0, n1, n2 = (w.detach().norm(dim=1, keepdim=True) for w in (w0, w1, w2))
    outs = []
    out_pos = 0
    for start, end, update, apply in ttt_ua_order:
        if update:
            _rec(trace, "update", start, end)
            ki, vi = k[:, start:end], v[:, start:end]
            g = mm(ki, w0)
            h = mm(ki, w2)
            hidden = F.silu(g) * h
            dhidden = mm(vi, w1.transpose(-1, -2))
            dh2 = dhidden * F.silu(g)
            dg = silu_backprop(dhidden * h, g)
            g1 = newton_schulz(mm((hidden * lr1[:, start:end]).transpose(-1, -2), vi), muon_update_steps)
            g0 = newton_schulz(mm((ki * lr0[:, start:end]).transpose(-1, -2), dg), muon_update_steps)
            g2 = newton_schulz(mm((ki * lr2[:, start:end]).transpose(-1, -2), dh2), muon_update_steps)
            w1, w0, w2 = w1 + g1, w0 + g0, w2 + g2
            w0 = w0 / (w0.norm(dim=1, keepdim=True) + 1e-5) * n0
            w1 = w1 / (w1.norm(dim=1, keepdim=True) + 1e-5) * n1
            w2 = w2 / (w2.norm(dim=1, keepdim=True) + 1e-5) * n2
        if apply:
            if trace is not None:
                trace.append(("apply", int(start), int(min(end, q.shape[1])), out_pos))
            qi = q[:, start:end]
            outs.append(mm(F.silu(mm(qi, w0)) * mm(qi, w2), w1))
            out_pos += qi.shape[1]
    return torch.cat(outs, dim=1), w0, w1, w2


def ar_mini_batch(
    w0, w1, w2, q, k, v, lr0, lr1, lr2, w_scale, num_repeat=1, mini_batch_size=-1, update_length=-1,
    update_every=-1, use_moun=False, num_moun_iters=3, weight_norm=True, fw_momentum=None, use_momentum=False,
    *, nm: Numerics = Numerics(), trace: Optional[list] = None, ns=None,
):
    """Autoregressive-video training driver (update-then-apply with an `update_every` stride).
    `ns` replaces the Newton-Schulz function (default: the reference's eager arithmetic, `newton_schulz`).

    Without momentum: lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:22-168 (the
    `num_repeat` loop wraps the chunk loop).  With momentum:
    ar_lact_swa_repeat_sp.py:27-193 (which has no `num_repeat` loop: one pass).
    """
    ns = newton_schulz if ns is None else ns
    L = k.shape[1]
    if update_length == -1:
        update_length = L
    if mini_batch_size == -1:
        mini_batch_size = update_length
    if update_every == -1:
        update_every = mini_batch_size * 2
    n0, n1, n2 = (w.norm(dim=2, keepdim=True) for w in (w0, w1, w2))
    out = torch.zeros_like(q)
    first = update_every - mini_batch_size
    _rec(trace, "apply", 0, min(first, L))
    out[:, :first] = apply_ref(w0, w1, w2, q[:, :first], nm)
    if use_momentum:
        m0, m1, m2 = torch.zeros_like(w0), torch.zeros_like(w1), torch.zeros_like(w2)
    for _ in range(1 if use_momentum else num_repeat):
        for s in range(first, update_length, update_every):
            e = s + mini_batch_size
            _rec(trace, "update", s, min(e, L))
            dw0, dw1, dw2 = grads_ref(w0, w1, w2, k[:, s:e], v[:, s:e], lr0[:, s:e], lr1[:, s:e], lr2[:, s:e],
                                      nm, style="ar", w_scale=w_scale)
            if use_momentum:
                beta = fw_momentum[:, s:e].mean(dim=1, keepdim=True)
                dw0, dw1, dw2 = dw0 + m0 * beta, dw1 + m1 * beta, dw2 + m2 * beta
                m0, m1, m2 = dw0, dw1, dw2
            if use_moun:
                dw1 = ns(dw1, num_moun_iters)
                dw0 = ns(dw0, num_moun_iters)
                dw2 = ns(dw2, num_moun_iters)
            w1, w0, w2 = w1 + dw1, w0 + dw0, w2 + dw2
            if weight_norm:
                w0, w1, w2 = _renorm_outer(w0, n0), _renorm_outer(w1, n1), _renorm_outer(w2, n2)
            e = s + update_every
            _rec(trace, "apply", s, min(e, L))
            out[:, s:e] = apply_ref(w0, w1, w2, q[:, s:e], nm)
    return out, w0, w1, w2


def ar_mini_batch_inference(
    w0, w1, w2, q, k, v, lr0, lr1, lr2, w_scale, num_repeat=1, mini_batch_size=-1, do_update=False,
    use_moun=False, num_moun_iters=3, weight_norm=True, fw_momentum=None, dw0_momentum=None,
    dw1_momentum=None, dw2_momentum=None, use_momentum=False, with_momentum_api=False,
    *, nm: Numerics = Numerics(), trace: Optional[list] = None,
):
    """Autoregressive-video inference driver: at most `num_repeat` updates on the first
    mini-batch, then apply to every query token.

    lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:171-296 (4-tuple return) and
    ar_lact_swa_repeat_sp.py:196-339 (momentum state in and out, 7-tuple return).
    """
    L = k.shape[1]
    if mini_batch_size == -1:
        mini_batch_size = L
    n0, n1, n2 = (w.norm(dim=2, keepdim=True) for w in (w0, w1, w2))
    if dw0_momentum is None and use_momentum:
        dw0_momentum, dw1_momentum, dw2_momentum = torch.zeros_like(w0), torch.zeros_like(w1), torch.zeros_like(w2)
    if do_update:
        for _ in range(num_repeat):
            e = mini_batch_size
            _rec(trace, "update", 0, min(e, L))
            dw0, dw1, dw2 = grads_ref(w0, w1, w2, k[:, :e], v[:, :e], lr0[:, :e], lr1[:, :e], lr2[:, :e],
                                      nm, style="ar", w_scale=w_scale)
            if use_momentum:
                beta = fw_momentum[:, :e].mean(dim=1, keepdim=True)
                dw0 = dw0 + dw0_momentum * beta
                dw1 = dw1 + dw1_momentum * beta
                dw2 = dw2 + dw2_momentum * beta
                dw0_momentum, dw1_momentum, dw2_momentum = dw0, dw1, dw2
            if use_moun:
                dw1 = newton_schulz(dw1, num_moun_iters)
                dw0 = newton_schulz(dw0, num_moun_iters)
                dw2 = newton_schulz(dw2, num_moun_iters)
            w1, w0, w2 = w1 + dw1, w0 + dw0, w2 + dw2
            if weight_norm:
                w0, w1, w2 = _renorm_outer(w0, n0), _renorm_outer(w1, n1), _renorm_outer(w2, n2)
    _rec(trace, "apply", 0, L)
    out = apply_ref(w0, w1, w2, q, nm)
    if with_momentum_api:
        return out, w0, w1, w2, dw0_momentum, dw1_momentum, dw2_momentum
    return out, w0, w1, w2


# ----------------------------------------------------------------------------------------------
# kernel-rounding model of the general scan (what the CUDA path computes), LLM layout.
# ----------------------------------------------------------------------------------------------
@dataclasses.dataclass
class ScanConfig:
    """Semantic switches of the general scan; mirrors the C-ABI configuration struct."""

    use_muon: bool = False
    ns_steps: int = 5
    ns_const_coeffs: bool = False  # False: tuned 5-triple table (ns_steps must be 5)
    ns_concat: bool = False  # Newton-Schulz on cat([dw0, dw2], dim=1)
    ns_gram_right: bool = False  # square matrices: iterate on the transpose (NVS layout)
    renorm: str = "outer"  # "none" | "outer" (eps outside) | "inner" (eps inside sqrt)
    prenorm: bool = False
    prenorm_bf16: bool = False  # fused pre-norm: normalised weights are stored as bf16
    overwrite_quirk: bool = False  # bidirectional: w <- renorm(NS(dw) + dw)
    w_scale: float = 1.0
    fp32_mode: bool = False  # activations / operands in fp32 (no bf16 rounding outside NS)


def _ns_model(G, cfg: ScanConfig):
    steps = cfg.ns_steps if cfg.ns_const_coeffs else None
    if cfg.ns_gram_right and G.size(1) == G.size(2):
        return newton_schulz_folded(G.transpose(1, 2), steps, fold_norm=True).transpose(1, 2)
    return newton_schulz_folded(G, steps, fold_norm=True)


def scan_model(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps: Sequence[Tuple[str, int, int, int]], cfg: ScanConfig,
               momentum=None, m_init=None, out_len: Optional[int] = None):
    """Kernel-rounding model of the general scan.  `steps` = (kind, start, end, out_start).

    Returns (o, w0, w1, w2, (m0, m1, m2) or None).  In bf16 mode the arithmetic is that of
    `apply_fused` / `grads_fused`; in fp32 mode plain fp32.  Momentum, Newton-Schulz and the
    renormalisation follow the reference lines cited on the drivers above.
    """
    act = torch.float32 if cfg.fp32_mode else BF16
    H = w0.shape[1]
    w0, w1, w2 = w0.float(), w1.float(), w2.float()
    n0, n1, n2 = (w.norm(dim=2, keepdim=True) for w in (w0, w1, w2))
    w0m, w1m, w2m = w0, w1, w2
    wdt = torch.float32 if cfg.fp32_mode else BF16
    ms = None
    if momentum is not None:
        ms = [torch.zeros_like(w0), torch.zeros_like(w1), torch.zeros_like(w2)] if m_init is None else [t.float() for t in m_init]
    out_len = q.shape[1] if out_len is None else out_len
    out = torch.zeros(q.shape[0], out_len, w1.shape[1], dtype=act)
    l0, l1, l2 = lr0[..., 0], lr1[..., 0], lr2[..., 0]

    def norm_w(w, n):
        if cfg.renorm == "none":
            return w
        if cfg.renorm == "inner":
            return w * (1 / torch.sqrt(torch.sum(w * w, dim=2, keepdim=True) + 1e-5)) * n
        return w / (w.norm(dim=2, keepdim=True) + 1e-5) * n

    for kind, s, e, o in steps:
        w02b = torch.cat([w0, w2], dim=1).to(wdt)
        w1b = w1.to(wdt)
        if kind == "apply":
            out[:, o:o + (e - s)] = apply_fused(w02b, w1b, q[:, s:e].to(act))
            continue
        dw02, dw1 = grads_fused(w02b, w1b, k[:, s:e].to(act), v[:, s:e].to(act), l0[:, s:e], l1[:, s:e], l2[:, s:e],
                                cfg.w_scale)
        dw0, dw2 = dw02[:, :H], dw02[:, H:]
        if ms is not None:
            beta = momentum[:, s:e].float().mean(dim=1, keepdim=True)
            dw0, dw1, dw2 = dw0.float() + ms[0] * beta, dw1.float() + ms[1] * beta, dw2.float() + ms[2] * beta
            ms = [dw0, dw1, dw2]
        g0, g1, g2 = dw0, dw1, dw2
        if cfg.use_muon:
            g1 = _ns_model(dw1, cfg)
            if cfg.ns_concat:
                g02 = _ns_model(torch.cat([dw0, dw2], dim=1), cfg)
                g0, g2 = g02[:, :H], g02[:, H:]
            else:
                g0, g2 = _ns_model(dw0, cfg), _ns_model(dw2, cfg)
        if cfg.overwrite_quirk and cfg.use_muon:
            w0m, w1m, w2m = g0.float() + dw0.float(), g1.float() + dw1.float(), g2.float() + dw2.float()
        else:
            w0m, w1m, w2m = w0m + g0.float(), w1m + g1.float(), w2m + g2.float()
        w0, w1, w2 = norm_w(w0m, n0), norm_w(w1m, n1), norm_w(w2m, n2)
        if cfg.prenorm:
            if cfg.prenorm_bf16:
                w0, w1, w2 = w0.to(BF16).float(), w1.to(BF16).float(), w2.to(BF16).float()
        else:
            w0m, w1m, w2m = w0, w1, w2
    return out, w0, w1, w2, ms


# ----------------------------------------------------------------------------------------------
# metrics (fp64)
# ----------------------------------------------------------------------------------------------
def rel_max(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max|a - ref| / max|ref| in float64."""
    a, ref = a.double(), ref.double()
    return float((a - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def rel_fro(a: torch.Tensor, ref: torch.Tensor) -> float:
    """||a - ref||_F / ||ref||_F in float64."""
    a, ref = a.double(), ref.double()
    return float((a - ref).norm() / ref.norm().clamp_min(1e-30))


def cosine(a: torch.Tensor, ref: torch.Tensor) -> float:
    a, ref = a.double().flatten(), ref.double().flatten()
    return float(torch.dot(a, ref) / (a.norm() * ref.norm()).clamp_min(1e-30))


# ----------------------------------------------------------------------------------------------
# seeded synthetic inputs
# ----------------------------------------------------------------------------------------------
def make_inputs(B: int, L: int, D: int, H: int, seed: int = 0, act_dtype=torch.float32, lr_dtype=torch.float32):
    """q,k,v ~ N(0,1), q and k L2-normalised per token; W0,W2 = randn/sqrt(D), W1 = randn/sqrt(H);
    lr = softplus(N(-2,1)) x3; beta = sigmoid(N(0,1)).  Initialisation follows
    minimal_implementations/bidirectional_lact_layer.py:206-210 and
    lact_llm/lact_model/layer_lact_swiglu.py:214-222.
    """
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, L, D, generator=g)
    k = torch.randn(B, L, D, generator=g)
    v = torch.randn(B, L, D, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    w0 = torch.randn(B, H, D, generator=g) / D ** 0.5
    w1 = torch.randn(B, D, H, generator=g) / H ** 0.5
    w2 = torch.randn(B, H, D, generator=g) / D ** 0.5
    lr = F.softplus(torch.randn(B, L, 3, generator=g) - 2.0)
    lr0, lr1, lr2 = (t.contiguous().to(lr_dtype) for t in lr.chunk(3, dim=-1))
    beta = torch.sigmoid(torch.randn(B, L, 1, generator=g))
    return dict(w0=w0, w1=w1, w2=w2, q=q.to(act_dtype), k=k.to(act_dtype), v=v.to(act_dtype),
                lr0=lr0, lr1=lr1, lr2=lr2, momentum=beta)


# ---------------------------------------------------------------------------------------------------
# layer prologue (inputs of the recurrence)
# ---------------------------------------------------------------------------------------------------
def qkv_prologue(xq: torch.Tensor, xk: torch.Tensor, xv: torch.Tensor, n_heads: int, qkv_silu: bool = True,
                 v_silu: bool = True):
    """Fast-weight inputs of the LLM layer without RoPE (lact_llm/lact_model/layer_lact_swiglu.py:399-414):
    split [b, s, n_h*d] into heads merged with the batch ([(b n_h), s, d]), SiLU on q and k (and v unless
    `no_v_silu`), then the per-head `l2_norm` of q and k (ttt_operation.py:19-26): x / (||x|| + 1e-5) with the
    norm, the sum and the quotient each rounded to the input dtype (bf16 under the layer's autocast)."""
    def heads(t):
        b, s, nd = t.shape
        d = nd // n_heads
        return t.reshape(b, s, n_heads, d).permute(0, 2, 1, 3).reshape(b * n_heads, s, d)

    def l2n(x):
        return (x / (x.norm(dim=-1, keepdim=True) + 1e-5)).type(x.dtype)

    q, k, v = heads(xq), heads(xk), heads(xv)
    if qkv_silu:
        q, k = F.silu(q), F.silu(k)
        if v_silu:
            v = F.silu(v)
    return l2n(q).contiguous(), l2n(k).contiguous(), v.contiguous()


def rotary_tables(head_dim: int, n_positions: int, base: float = 500000.0, dtype=BF16):
    """cos / sin tables of `fla.modules.RotaryEmbedding(dim=head_dim, base=rope_theta)` (flash-linear-attention 0.5.1,
    `_update_cos_sin_cache`): inv_freq = 1 / base^(arange(0, dim, 2) / dim) in fp32, positions in fp32, outer product,
    cos / sin cast to the activations' dtype.  The reference layer builds it with base = rope_theta (default 500000,
    lact_llm/lact_model/layer_lact_swiglu.py:141, 170).  Returns (cos, sin), each [n_positions, head_dim / 2]."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(n_positions, dtype=torch.float32), inv_freq)
    return torch.cos(freqs).to(dtype), torch.sin(freqs).to(dtype)


def rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seqlen_offset: int = 0, policy: str = "ref"):
    """Rotary embedding of x [b, s, heads, head_dim] in the non-interleaved layout (first half pairs with second half).
    policy "ref": the arithmetic of fla's own PyTorch restatement `rotary_embedding_ref` (x * cos + rotate_half(x) *
    sin in x's dtype: every product and the sum rounded); policy "fused": fp32 products and sum from the bf16 inputs,
    one rounding (what a fused kernel does; the reference's Triton kernel computes in fp32 as well)."""
    s, hd = x.shape[1], x.shape[-1]
    c = cos[seqlen_offset:seqlen_offset + s]
    sn = sin[seqlen_offset:seqlen_offset + s]
    if policy == "ref":
        c2 = torch.cat([c, c], dim=-1)[:, None, :]
        s2 = torch.cat([sn, sn], dim=-1)[:, None, :]
        x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
        return x * c2 + torch.cat([-x2, x1], dim=-1) * s2
    xf, cf, sf = x.float(), c.float()[:, None, :], sn.float()[:, None, :]
    x1, x2 = xf[..., :hd // 2], xf[..., hd // 2:]
    return torch.cat([x1 * cf - x2 * sf, x1 * sf + x2 * cf], dim=-1).to(x.dtype)


def qkv_prologue_rope(xq, xk, xv, n_heads: int, rope_head_dim: int, cos, sin, seqlen_offset: int = 0,
                      qkv_silu: bool = True, v_silu: bool = True, policy: str = "ref", cu_seqlens=None):
    """`qkv_prologue` followed by the rotary embedding of fast q and k as the layer applies it when `ttt_nope` is off
    (lact_llm/lact_model/layer_lact_swiglu.py:417-446): fast-weight heads merged back to [b, s, n_h * d], re-split
    into attention heads of `rope_head_dim` features, rotated, and split into fast-weight heads again."""
    if cu_seqlens is not None:   # packed sequences (batch of one): positions restart at every sequence start
        cu = [int(c) for c in cu_seqlens]
        parts = [qkv_prologue_rope(xq[:, a:e], xk[:, a:e], xv[:, a:e], n_heads, rope_head_dim, cos, sin, seqlen_offset,
                                   qkv_silu, v_silu, policy) for a, e in zip(cu[:-1], cu[1:])]
        return tuple(torch.cat([p[i] for p in parts], dim=1) for i in range(3))
    q, k, v = qkv_prologue(xq, xk, xv, n_heads, qkv_silu, v_silu)
    b, s, nd = xq.shape
    d = nd // n_heads

    def rot(t):
        merged = t.reshape(b, n_heads, s, d).permute(0, 2, 1, 3).reshape(b, s, nd)
        r = rotary(merged.reshape(b, s, nd // rope_head_dim, rope_head_dim), cos, sin, seqlen_offset, policy)
        return r.reshape(b, s, n_heads, d).permute(0, 2, 1, 3).reshape(b * n_heads, s, d).contiguous()

    return rot(q), rot(k), v


def lr_prologue(lr_proj: torch.Tensor, n_heads: int, base_lr: float, momentum_logits: Optional[torch.Tensor] = None):
    """Per-token learning rates and momentum of the LLM layer (lact_llm/lact_model/layer_lact_swiglu.py:463-480 and
    245-249): lr = softplus(lr_proj.float() + inv_softplus(base_lr)) ([b, s, n_h * 3], three per head), split into
    three [(b n_h), s, 1] fp32 tensors; momentum = sigmoid of the projection in its own dtype (bf16 under autocast),
    then .float(), as [(b n_h), s, 1]."""
    import math
    b, s, n3 = lr_proj.shape
    base_lr_inv = base_lr + math.log(-math.expm1(-base_lr))  # inv_softplus, layer_lact_swiglu.py:44-49
    lr = F.softplus(lr_proj.float() + base_lr_inv)
    lr = lr.reshape(b, s, n_heads, 3).permute(0, 2, 1, 3).reshape(b * n_heads, s, 3)
    outs = [lr[..., i:i + 1].contiguous() for i in range(3)]
    mom = None
    if momentum_logits is not None:
        m = torch.sigmoid(momentum_logits).float()
        mom = m.reshape(b, s, n_heads, 1).permute(0, 2, 1, 3).reshape(b * n_heads, s, 1).contiguous()
    return outs[0], outs[1], outs[2], mom


def out_epilogue(fw_x: torch.Tensor, weight: torch.Tensor, n_heads: int, scale_proj: Optional[torch.Tensor] = None,
                 o_attn: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    """Output side of the LLM layer (lact_llm/lact_model/layer_lact_swiglu.py:556-568): per-head RMSNorm of the
    recurrence's output fw_x [(b n_h), s, d] (the reference uses `fla.modules.RMSNorm`, flash-linear-attention 0.5.1,
    a Triton kernel whose arithmetic is x * rsqrt(mean(x^2) + eps) * weight in fp32, rounded to x's dtype), times the
    gate silu(scale_proj) (both bf16 under autocast, product rounded), heads merged back to [b, s, n_h * d] and
    added to the attention output."""
    B, s, d = fw_x.shape
    b = B // n_heads
    xf = fw_x.float()
    y = (xf * (1 / torch.sqrt(xf.square().mean(dim=-1, keepdim=True) + eps)) * weight.float()).to(fw_x.dtype)
    if scale_proj is not None:
        gate = F.silu(scale_proj).reshape(b, s, n_heads, d).permute(0, 2, 1, 3).reshape(B, s, d)
        y = y * gate
    y = y.reshape(b, n_heads, s, d).permute(0, 2, 1, 3).reshape(b, s, n_heads * d)
    return (o_attn + y) if o_attn is not None else y.contiguous()



def sliding_window_attention(q, k, v, window_size=None, softmax_scale=None, block: int = 1024, cu_seqlens=None):
    """Causal attention over the keys (i - window_size, i] in fp32: the published semantics of
    `flash_attn_func(q, k, v, causal=True, window_size=(window_size - 1, 0))` (flash-attn 2.x: a query attends keys
    [i - left, i + right]), the call the reference makes at lact_llm/lact_model/layer_lact_swiglu.py:386-394 and
    minimal_implementations/causal_lact_with_sliding_window_attn.py:380-384.  flash-attn has no CPU implementation,
    so this restatement is checked against `torch.nn.functional.scaled_dot_product_attention` with the same band
    mask (tests/test_oracle_golden.py).  q, k, v: [b, l, h, d]; returns fp32 [b, l, h, d]."""
    if cu_seqlens is not None:   # sequences packed into one batch entry (flash_attn_varlen_func): one by one
        cu = [int(c) for c in cu_seqlens]
        return torch.cat([sliding_window_attention(q[:, s0:s1], k[:, s0:s1], v[:, s0:s1], window_size, softmax_scale, block)
                          for s0, s1 in zip(cu[:-1], cu[1:])], dim=1)
    b, l, h, d = q.shape
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    w = l if not window_size else int(window_size)
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))  # [b, h, l, d]
    out = torch.empty(b, h, l, d)
    for s0 in range(0, l, block):
        s1 = min(l, s0 + block)
        k0 = max(0, s0 - (w - 1))
        sc = torch.matmul(qf[:, :, s0:s1], kf[:, :, k0:s1].transpose(-1, -2)) * scale
        i = torch.arange(s0, s1).view(-1, 1)
        j = torch.arange(k0, s1).view(1, -1)
        sc = sc.masked_fill(~((j <= i) & (j > i - w)), float("-inf"))
        out[:, :, s0:s1] = torch.matmul(torch.softmax(sc, dim=-1), vf[:, :, k0:s1])
    return out.permute(0, 2, 1, 3).contiguous()


def masked_attention(q, k, v, visible, softmax_scale=None):
    """fp32 softmax attention with an explicit boolean visibility matrix `visible` [lq, lk] (True = the query may
    attend the key), q [b, lq, h, d], k, v [b, lk, h, d] -> fp32 [b, lq, h, d].  The definition the block-attention
    restatements below are written against."""
    d = q.shape[-1]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    sc = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    sc = sc.masked_fill(~visible.view(1, 1, *visible.shape), float("-inf"))
    return torch.matmul(torch.softmax(sc, dim=-1), vf).permute(0, 2, 1, 3).contiguous()


def ar_block_visibility(l, mini_batch_size, update_every, num_chunks, kv_cache_size, repeated):
    """Which key every query of the autoregressive-video layer's attention sees, as ONE [l, l] matrix, from the
    structure of lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:299-365 (`repeated` False) and :368-463
    (True): the leading update_every - mini_batch_size tokens attend among themselves (as num_repeat separate blocks
    when repeated); in every later block of update_every tokens the first mini_batch_size (clean) tokens attend among
    themselves and the noisy tokens attend over the last kv_cache_size clean keys plus - not repeated - the
    mini_batch_size keys after them, or - repeated - the keys of their own mini_batch_size block."""
    mb, ue = mini_batch_size, update_every
    first = ue - mb
    assert l == first + ue * (num_chunks - 1)
    vis = torch.zeros(l, l, dtype=torch.bool)
    if repeated:
        for s in range(0, first, mb):
            vis[s:s + mb, s:s + mb] = True
    else:
        vis[:first, :first] = True
    for c in range(num_chunks - 1):
        s = first + c * ue
        vis[s:s + mb, s:s + mb] = True
        if repeated:
            for r in range(ue // mb - 1):
                n0 = s + mb + r * mb
                vis[n0:n0 + mb, s + mb - kv_cache_size:s + mb] = True
                vis[n0:n0 + mb, n0:n0 + mb] = True
        else:
            vis[s + mb:s + ue, s + mb - kv_cache_size:min(s + ue, s + 2 * mb)] = True
    return vis
