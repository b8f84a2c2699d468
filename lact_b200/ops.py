"""Drop-in replacements for the reference's fused sub-ops and chunk drivers.

Same names, positional order, keyword defaults and return types as the reference functions
(cited per function); the arithmetic runs in the sm_100a kernels of liblact_b200.so through the
C ABI.  bf16 activations run the fused tcgen05 program (with a training backward); fp32 activations
run the accuracy path of `fp32_mode` (forward only).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib as L
from . import program as P

BF16 = torch.bfloat16


def _no_trace(fn):
    """The ops are ctypes calls into a CUDA library: TorchDynamo must not trace into them.  The
    reference wraps its functions in @torch.compile; a caller that compiles its layer gets a graph
    break around these calls instead of a tracing error."""
    disable = getattr(getattr(torch, "compiler", None), "disable", None)
    return disable(fn) if disable is not None else fn


def _need_cuda(*ts: torch.Tensor) -> torch.device:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("lact_b200 runs on CUDA tensors only (there is no CPU implementation)")
        if dev is not None and t.device != dev:
            raise ValueError("all tensors must be on the same device")
        dev = t.device
    return dev


def _act(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != BF16:
        raise TypeError(f"{name} must be bfloat16, or q, k, v all float32 (got {t.dtype})")
    if t.dim() != 3:
        raise ValueError(f"{name} must be [b, l, d]")
    if t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def _vec(t: torch.Tensor, B: int, Ltok: int, name: str) -> torch.Tensor:
    """[b, l, 1] or [b, l] per-token scalar -> contiguous [b, l] in fp32 or bf16."""
    if t.dim() == 3:
        if t.shape[2] != 1:
            raise ValueError(f"{name} must be [b, l, 1]")
        t = t[..., 0]
    if tuple(t.shape) != (B, Ltok):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {(B, Ltok)}")
    if t.dtype not in (torch.float32, BF16):
        t = t.float()
    return t.contiguous()


def _weight(t: torch.Tensor, shape: tuple, name: str) -> torch.Tensor:
    if tuple(t.shape) != shape:
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
    if t.dtype not in (torch.float32, BF16):
        t = t.float()
    return t.contiguous()


def scan_eager(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps: Sequence[P.Step], *, out_len: Optional[int] = None,
               momentum=None, m_init=None, use_muon=False, ns_steps=5, ns_const_coeffs=False, ns_concat=False,
               ns_gram_right=False, renorm=L.RENORM_EPS_OUTSIDE, prenorm=False, prenorm_bf16=False,
               overwrite_quirk=False, w_scale=1.0, return_state=False, return_momentum=False, _state_dump=None,
               _ns_trace=None):
    """Forward of the general chunk recurrence, straight through the C ABI (`lact_scan_fwd`), no
    autograd.  `scan` is the public, differentiable and compilable entry point."""
    dev = _need_cuda(w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum)
    if q.dtype == k.dtype == v.dtype == torch.float32:
        return _scan_f32(dev, w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, out_len, momentum, m_init,
                         dict(use_muon=use_muon, ns_steps=ns_steps, ns_const_coeffs=ns_const_coeffs,
                              ns_concat=ns_concat, ns_gram_right=ns_gram_right, renorm=renorm, prenorm=prenorm,
                              prenorm_bf16=prenorm_bf16, overwrite_quirk=overwrite_quirk, w_scale=w_scale,
                              return_state=return_state, return_momentum=return_momentum), _state_dump)
    q, k, v = _act(q, "q"), _act(k, "k"), _act(v, "v")
    B, Ltok, D = k.shape
    H = w0.shape[1]
    if q.shape[0] != B or q.shape[2] != D or v.shape != k.shape:
        raise ValueError("q, k, v shapes disagree")
    w0 = _weight(w0, (B, H, D), "w0")
    w1 = _weight(w1, (B, D, H), "w1")
    w2 = _weight(w2, (B, H, D), "w2")
    if not (w0.dtype == w1.dtype == w2.dtype):
        w0, w1, w2 = w0.float(), w1.float(), w2.float()
    lr0, lr1, lr2 = (_vec(t, B, Ltok, n) for t, n in ((lr0, "lr0"), (lr1, "lr1"), (lr2, "lr2")))
    if not (lr0.dtype == lr1.dtype == lr2.dtype):
        lr0, lr1, lr2 = lr0.float(), lr1.float(), lr2.float()
    if momentum is not None:
        momentum = _vec(momentum, B, Ltok, "momentum")
    if q.shape[1] != Ltok:
        raise ValueError("q and k must have the same number of tokens")
    out_len = Ltok if out_len is None else int(out_len)
    # The reference drivers start from torch.zeros_like(q): tokens no APPLY step covers stay zero (e.g. the tail
    # beyond update_length of the autoregressive-video drivers).  Zero-filling costs a full pass over o, so it is
    # done only when the program leaves a gap.
    covered, full = 0, True
    for s_ in sorted((int(st[3]), int(st[3]) + int(st[2]) - int(st[1])) for st in steps if st[0] == P.APPLY):
        if s_[0] > covered:
            full = False
            break
        covered = max(covered, s_[1])
    full = full and covered >= out_len
    o = (torch.empty if full else torch.zeros)(B, out_len, D, dtype=BF16, device=dev)

    cfg = L.ScanConfig()
    cfg.B, cfg.L, cfg.D, cfg.H, cfg.out_len = B, Ltok, D, H, out_len
    cfg.act_dtype = L.LACT_BF16
    cfg.lr_dtype = L.dtype_code(lr0)
    cfg.mom_dtype = L.dtype_code(momentum) if momentum is not None else L.LACT_F32
    cfg.w_dtype = L.dtype_code(w0)
    cfg.use_momentum = int(momentum is not None)
    cfg.use_muon, cfg.ns_steps, cfg.ns_const_coeffs = int(use_muon), int(ns_steps), int(ns_const_coeffs)
    cfg.ns_concat, cfg.ns_gram_right = int(ns_concat), int(ns_gram_right)
    cfg.renorm, cfg.prenorm, cfg.prenorm_bf16 = int(renorm), int(prenorm), int(prenorm_bf16)
    cfg.overwrite_quirk, cfg.w_scale = int(overwrite_quirk), float(w_scale)
    cfg.q_bs, cfg.q_ts = q.stride(0), q.stride(1)
    cfg.k_bs, cfg.k_ts = k.stride(0), k.stride(1)
    cfg.v_bs, cfg.v_ts = v.stride(0), v.stride(1)
    cfg.o_bs, cfg.o_ts = o.stride(0), o.stride(1)

    n = len(steps)
    kind = (C.c_int32 * n)(*[s[0] for s in steps])
    start = (C.c_int64 * n)(*[s[1] for s in steps])
    end = (C.c_int64 * n)(*[s[2] for s in steps])
    outs = (C.c_int64 * n)(*[s[3] for s in steps])
    lib = L.lib()
    need = C.c_size_t(0)
    L.check(lib.lact_scan_workspace_bytes(C.byref(cfg), n, kind, start, end, C.byref(need)), "lact_scan_workspace_bytes")
    ws = L.workspace(need.value, dev)

    io = L.ScanIO()
    io.w0, io.w1, io.w2 = w0.data_ptr(), w1.data_ptr(), w2.data_ptr()
    io.q, io.k, io.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    io.lr0, io.lr1, io.lr2 = lr0.data_ptr(), lr1.data_ptr(), lr2.data_ptr()
    io.momentum = momentum.data_ptr() if momentum is not None else None
    keep = []
    if m_init is not None:
        m_init = [t.float().contiguous() for t in m_init]
        keep += m_init
        io.m0_in, io.m1_in, io.m2_in = (t.data_ptr() for t in m_init)
    io.o = o.data_ptr()
    if _state_dump is not None:
        io.state_dump = _state_dump.data_ptr()
    if _ns_trace is not None:
        io.ns_trace = _ns_trace.data_ptr()
    state = mom = None
    if return_state:
        state = (torch.empty(B, H, D, dtype=torch.float32, device=dev),
                 torch.empty(B, D, H, dtype=torch.float32, device=dev),
                 torch.empty(B, H, D, dtype=torch.float32, device=dev))
        io.w0_out, io.w1_out, io.w2_out = (t.data_ptr() for t in state)
    if return_momentum:
        mom = (torch.empty(B, H, D, dtype=torch.float32, device=dev),
               torch.empty(B, D, H, dtype=torch.float32, device=dev),
               torch.empty(B, H, D, dtype=torch.float32, device=dev))
        io.m0_out, io.m1_out, io.m2_out = (t.data_ptr() for t in mom)
    with torch.cuda.device(dev):
        L.check(lib.lact_scan_fwd(C.byref(cfg), C.byref(io), n, kind, start, end, outs, ws.data_ptr(), ws.numel(),
                                  L.stream_ptr()), "lact_scan_fwd")
    L.mark_pending(ws)
    res = [o]
    if return_state:
        res.extend(state)
    if return_momentum:
        res.extend(mom)
    return res[0] if len(res) == 1 else tuple(res)


def ns_trace_layout(B, Ltok, D, H, opts) -> Tuple[int, int]:
    """(bytes of Newton-Schulz trace the training forward keeps per update, offset of the w1 group's trace), or
    (0, 0) when this configuration keeps none (Muon off, more than five iterations)."""
    if not opts.get("use_muon"):
        return 0, 0
    cfg = L.ScanConfig()
    cfg.B, cfg.L, cfg.D, cfg.H, cfg.out_len = B, Ltok, D, H, Ltok
    cfg.act_dtype = L.LACT_BF16
    cfg.use_muon, cfg.ns_steps = 1, int(opts.get("ns_steps", 5))
    cfg.ns_const_coeffs, cfg.ns_concat = int(bool(opts.get("ns_const_coeffs"))), int(bool(opts.get("ns_concat")))
    cfg.ns_gram_right, cfg.renorm = int(bool(opts.get("ns_gram_right"))), int(opts.get("renorm", L.RENORM_EPS_OUTSIDE))
    stride, off = C.c_size_t(0), C.c_size_t(0)
    rc = L.lib().lact_scan_ns_trace_bytes(C.byref(cfg), C.byref(stride), C.byref(off))
    if rc != 0:
        return 0, 0
    return int(stride.value), int(off.value)


def _scan_f32(dev, w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, out_len, momentum, m_init, opts, state_dump):
    """fp32 activations: validate as `scan` does and run the step program in `fp32_mode`."""
    from .fp32_mode import scan_f32
    if state_dump is not None:
        raise NotImplementedError("the per-update state dump is a bf16-mode feature")
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        if t.dim() != 3:
            raise ValueError(f"{name} must be [b, l, d]")
    B, Ltok, D = k.shape
    H = w0.shape[1]
    if q.shape[0] != B or q.shape[2] != D or v.shape != k.shape or q.shape[1] != Ltok:
        raise ValueError("q, k, v shapes disagree")
    w0, w1, w2 = _weight(w0, (B, H, D), "w0"), _weight(w1, (B, D, H), "w1"), _weight(w2, (B, H, D), "w2")
    lr0, lr1, lr2 = (_vec(t, B, Ltok, n).float() for t, n in ((lr0, "lr0"), (lr1, "lr1"), (lr2, "lr2")))
    if momentum is not None:
        momentum = _vec(momentum, B, Ltok, "momentum")
    return scan_f32(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, out_len=out_len, momentum=momentum, m_init=m_init,
                    **opts)


# ----------------------------------------------------------------------------------------------
# registered operators: the recurrence as `torch.ops.lact_b200.scan_fwd` / `scan_bwd`
# ----------------------------------------------------------------------------------------------
# The reference wraps its functions in @torch.compile.  TorchDynamo cannot trace ctypes calls, so
# the recurrence is registered as a custom operator with a fake (shape-only) implementation and
# an autograd formula: a compiled caller sees one opaque node, without a graph break.
# cfg = [use_muon, ns_steps, ns_const_coeffs, ns_concat, ns_gram_right, renorm, prenorm,
#        prenorm_bf16, overwrite_quirk, detach_norms, out_len (-1: all tokens), return_momentum, save]
_CFG_KEYS = ("use_muon", "ns_steps", "ns_const_coeffs", "ns_concat", "ns_gram_right", "renorm", "prenorm",
             "prenorm_bf16", "overwrite_quirk")


def _opts_of(cfg: Sequence[int], w_scale: float) -> dict:
    d = {k_: int(cfg[i]) for i, k_ in enumerate(_CFG_KEYS)}
    for k_ in ("use_muon", "ns_const_coeffs", "ns_concat", "ns_gram_right", "prenorm", "prenorm_bf16", "overwrite_quirk"):
        d[k_] = bool(d[k_])
    d["w_scale"] = float(w_scale)
    return d


def _steps_of(flat: Sequence[int]) -> List[P.Step]:
    return [tuple(int(x) for x in flat[i:i + 4]) for i in range(0, len(flat), 4)]


@torch.library.custom_op("lact_b200::scan_fwd", mutates_args=(), device_types="cuda")
def _scan_fwd_op(w0: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, q: torch.Tensor, k: torch.Tensor,
                 v: torch.Tensor, lr0: torch.Tensor, lr1: torch.Tensor, lr2: torch.Tensor,
                 momentum: Optional[torch.Tensor], m0: Optional[torch.Tensor], m1: Optional[torch.Tensor],
                 m2: Optional[torch.Tensor], steps: List[int], cfg: List[int], w_scale: float) -> List[torch.Tensor]:
    """[o, w0', w1', w2'] (+ [m0', m1', m2'] if cfg[11]) (+ [saved state] if cfg[12])."""
    opts, st = _opts_of(cfg, w_scale), _steps_of(steps)
    out_len = None if cfg[10] < 0 else int(cfg[10])
    if cfg[12]:
        from .backward import scan_forward_saving
        opts["out_len"] = out_len
        o, a, b, c, dump, ns_dump = scan_forward_saving(opts, st, w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum)
        return [o, a, b, c, dump, ns_dump]
    m_init = (m0, m1, m2) if m0 is not None else None
    res = scan_eager(w0, w1, w2, q, k, v, lr0, lr1, lr2, st, out_len=out_len, momentum=momentum, m_init=m_init,
                     return_state=True, return_momentum=bool(cfg[11]), **opts)
    return list(res)


@_scan_fwd_op.register_fake
def _scan_fwd_fake(w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum, m0, m1, m2, steps, cfg, w_scale):
    B, Ltok, D = k.shape
    H = w0.shape[1]
    out_len = Ltok if cfg[10] < 0 else int(cfg[10])
    f32 = torch.float32
    outs = [q.new_empty((B, out_len, D)), q.new_empty((B, H, D), dtype=f32), q.new_empty((B, D, H), dtype=f32),
            q.new_empty((B, H, D), dtype=f32)]
    if cfg[11]:
        outs += [q.new_empty((B, H, D), dtype=f32), q.new_empty((B, D, H), dtype=f32), q.new_empty((B, H, D), dtype=f32)]
    if cfg[12]:
        n_upd = sum(1 for i in range(0, len(steps), 4) if steps[i] == P.UPDATE)
        outs.append(q.new_empty((max(n_upd, 1), 2 * (B * 2 * H * D + B * D * H)), dtype=f32))
        stride, _ = ns_trace_layout(B, Ltok, D, H, _opts_of(cfg, w_scale))
        outs.append(q.new_empty((max(n_upd, 1) * stride if stride else 1,), dtype=torch.uint8))
    return outs


@torch.library.custom_op("lact_b200::scan_bwd", mutates_args=(), device_types="cuda")
def _scan_bwd_op(w0: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, q: torch.Tensor, k: torch.Tensor,
                 v: torch.Tensor, lr0: torch.Tensor, lr1: torch.Tensor, lr2: torch.Tensor,
                 momentum: Optional[torch.Tensor], dump: torch.Tensor, ns_dump: torch.Tensor, wf0: torch.Tensor,
                 wf1: torch.Tensor, wf2: torch.Tensor, dO: torch.Tensor, gw0: Optional[torch.Tensor],
                 gw1: Optional[torch.Tensor], gw2: Optional[torch.Tensor], steps: List[int], cfg: List[int],
                 w_scale: float) -> List[torch.Tensor]:
    """Gradients of (w0, w1, w2, q, k, v, lr0, lr1, lr2[, momentum]) from the cotangents of o (dO) and,
    optionally, of the returned final fast weights (gw0, gw1, gw2)."""
    from .backward import scan_backward
    opts = _opts_of(cfg, w_scale)
    opts["_detach_norms"] = bool(cfg[9])
    gwf = (gw0, gw1, gw2) if (gw0 is not None or gw1 is not None or gw2 is not None) else None
    g = scan_backward(opts, _steps_of(steps), w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum, dump, wf0, wf1, wf2,
                      dO.contiguous(), gwf, ns_dump if ns_dump.numel() > 1 else None)
    # operator outputs must not alias each other: the w0 / w2 gradients are two halves of one buffer (copied); the
    # others are fresh tensors of the sweep
    g = [t for t in g if t is not None]
    return [g[0].clone(memory_format=torch.contiguous_format), g[1], g[2].clone(memory_format=torch.contiguous_format)] + \
           [t if t.is_contiguous() else t.contiguous() for t in g[3:]]


@_scan_bwd_op.register_fake
def _scan_bwd_fake(w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum, dump, ns_dump, wf0, wf1, wf2, dO, gw0, gw1, gw2,
                   steps, cfg, w_scale):
    outs = [torch.empty_like(t) for t in (w0, w1, w2, q, k, v, lr0, lr1, lr2)]
    if momentum is not None:
        outs.append(torch.empty_like(momentum))
    return outs


def _scan_setup_context(ctx, inputs, output):
    w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum, m0, m1, m2, steps, cfg, w_scale = inputs
    ctx.steps, ctx.cfg, ctx.w_scale, ctx.has_momentum, ctx.saved = list(steps), list(cfg), float(w_scale), momentum is not None, bool(cfg[12])
    # unused outputs (the final weights when the caller drops them, the saved-state buffer always) must not
    # arrive in the backward as materialised zero tensors: the saved state alone is gigabytes
    ctx.set_materialize_grads(False)
    if cfg[12]:
        keep = [w0, w1, w2, q, k, v, lr0, lr1, lr2] + ([momentum] if momentum is not None else []) + \
               [output[4], output[5], output[1], output[2], output[3]]
        ctx.save_for_backward(*keep)


def _scan_autograd(ctx, grads):
    if not ctx.saved:
        raise RuntimeError("lact_b200::scan_fwd was run without saving state for backward")
    t = list(ctx.saved_tensors)
    ins, rest = t[:9], t[9:]
    momentum = rest.pop(0) if ctx.has_momentum else None
    dump, ns_dump, wf0, wf1, wf2 = rest
    dO = grads[0]
    if dO is None:
        q, k = ins[3], ins[4]
        dO = q.new_zeros((q.shape[0], ctx.cfg[10] if ctx.cfg[10] >= 0 else k.shape[1], q.shape[2]))
    # cotangents of the returned final weights (None when the caller did not use them)
    gw = [g_.float().contiguous() if g_ is not None else None for g_ in grads[1:4]]
    g = torch.ops.lact_b200.scan_bwd(*ins, momentum, dump, ns_dump, wf0, wf1, wf2, dO, gw[0], gw[1], gw[2], ctx.steps,
                                     ctx.cfg, ctx.w_scale)
    dmom = g[9] if ctx.has_momentum else None
    return (*g[:9], dmom, None, None, None, None, None, None)


_scan_fwd_op.register_autograd(_scan_autograd, setup_context=_scan_setup_context)


def scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps: Sequence[P.Step], *, out_len: Optional[int] = None,
         momentum=None, m_init=None, use_muon=False, ns_steps=5, ns_const_coeffs=False, ns_concat=False,
         ns_gram_right=False, renorm=L.RENORM_EPS_OUTSIDE, prenorm=False, prenorm_bf16=False, overwrite_quirk=False,
         w_scale=1.0, return_state=False, return_momentum=False, _detach_norms=False):
    """General chunk recurrence in the LLM layout (w0, w2: [B,H,D]; w1: [B,D,H]); see
    `lact_scan_fwd` in include/lact_b200.h.  Returns o, and optionally the final fast weights
    and momentum state (fp32).  Runs as the registered operator `lact_b200::scan_fwd`; when
    gradients are enabled and an input requires grad, its autograd formula (`backward.py`) applies."""
    tensors = (w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum)
    save = torch.is_grad_enabled() and any(torch.is_tensor(t) and t.requires_grad for t in tensors)
    if save:
        if m_init is not None or return_momentum:
            raise NotImplementedError("gradients through a momentum state passed in / returned are not implemented")
        if q.dtype == torch.float32:
            raise NotImplementedError("fp32 mode is forward only; the training backward runs on bf16 activations")
        if prenorm and overwrite_quirk:
            raise NotImplementedError("no reference recurrence combines pre-norm with the bidirectional overwrite")
    cfg = [int(use_muon), int(ns_steps), int(ns_const_coeffs), int(ns_concat), int(ns_gram_right), int(renorm),
           int(prenorm), int(prenorm_bf16), int(overwrite_quirk), int(_detach_norms),
           -1 if out_len is None else int(out_len), int(return_momentum), int(save)]
    flat = [int(x) for s_ in steps for x in s_]
    m = tuple(m_init) if m_init is not None else (None, None, None)
    res = torch.ops.lact_b200.scan_fwd(w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum, m[0], m[1], m[2], flat, cfg,
                                       float(w_scale))
    out = [res[0]]
    if return_state:
        out += list(res[1:4])
    if return_momentum:
        out += list(res[4:7])
    return out[0] if len(out) == 1 else tuple(out)


# ----------------------------------------------------------------------------------------------
# chunk drivers, reference signatures
# ----------------------------------------------------------------------------------------------
def block_causal_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size: int = 2048, use_muon: bool = False,
                             momentum: torch.Tensor = None):
    """lact_llm/lact_model/ttt_operation.py:69-214: causal apply-then-update recurrence, post-norm,
    Newton-Schulz per matrix, renorm with eps outside the norm.  Returns o [b, l, dv]."""
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, P.causal_program(k.shape[1], chunk_size), momentum=momentum,
                use_muon=use_muon, renorm=L.RENORM_EPS_OUTSIDE)


def prenorm_block_causal_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size: int = 2048,
                                     use_muon: bool = False, momentum: torch.Tensor = None):
    """lact_llm/lact_model/ttt_operation.py:217-364: as above with an un-normalised master copy."""
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, P.causal_program(k.shape[1], chunk_size), momentum=momentum,
                use_muon=use_muon, renorm=L.RENORM_EPS_OUTSIDE, prenorm=True)


def minimal_block_causal_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, momentum: torch.Tensor = None,
                                     use_muon: bool = True, chunk_size: int = 2048):
    """minimal_implementations/causal_lact_with_sliding_window_attn.py:83-211 (note the different
    order and defaults of the last three arguments)."""
    return block_causal_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size=chunk_size, use_muon=use_muon,
                                    momentum=momentum)


def postnorm_block_causal_lact_swiglu_fused_kernel_triton(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size: int = 2048,
                                                          use_muon: bool = False, momentum: torch.Tensor = None):
    """lact_llm/lact_model/ttt_operation_fused_kernel.py:66-186: Newton-Schulz on the concatenated
    [2H, D] gradient, renorm with eps inside the square root."""
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, P.causal_program(k.shape[1], chunk_size), momentum=momentum,
                use_muon=use_muon, ns_concat=True, renorm=L.RENORM_EPS_INSIDE)


def prenorm_block_causal_lact_swiglu_fused_kernel_triton(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size: int = 2048,
                                                         use_muon: bool = False, momentum: torch.Tensor = None):
    """lact_llm/lact_model/ttt_operation_fused_kernel.py:189-316: fp32 master, bf16 normalised copy."""
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, P.causal_program(k.shape[1], chunk_size), momentum=momentum,
                use_muon=use_muon, ns_concat=True, renorm=L.RENORM_EPS_OUTSIDE, prenorm=True, prenorm_bf16=True)


def bidirectional_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, use_muon: bool = True) -> torch.Tensor:
    """minimal_implementations/bidirectional_lact_layer.py:73-160, including its behaviour with
    Muon: w <- renorm(NS(dw) + dw)."""
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, P.bidirectional_program(k.shape[1]), use_muon=use_muon,
                renorm=L.RENORM_EPS_OUTSIDE, overwrite_quirk=True)


def fast_weight_swish_glu_weight_norm_mini_batch_apply(w0, w1, w2, q, k, v, lr0, lr1, lr2, ttt_ua_order: list,
                                                       muon_update_steps: int = 0):
    """lact_nvs/lact_ttt.py:70-147.  NVS layout: w0, w2 [b, d, dh], w1 [b, dh, d].  Returns
    (output, w0, w1, w2) with the weights in the same layout (fp32)."""
    steps, out_len = P.operator_list_program([tuple(op) for op in ttt_ua_order], k.shape[1])
    t = lambda w: w.transpose(1, 2)
    o, a, b, c = scan(t(w0), t(w1), t(w2), q, k, v, lr0, lr1, lr2, steps, out_len=out_len, use_muon=True,
                      ns_steps=int(muon_update_steps), ns_const_coeffs=True, ns_gram_right=True,
                      renorm=L.RENORM_EPS_OUTSIDE, return_state=True, _detach_norms=True)
    return o, t(a).contiguous(), t(b).contiguous(), t(c).contiguous()


def ar_fast_weight_swish_glu_weight_norm_mini_batch(w0, w1, w2, q, k, v, lr0, lr1, lr2, w_scale: float,
                                                    num_repeat: int = 1, mini_batch_size: int = -1,
                                                    update_length: int = -1, update_every: int = -1,
                                                    use_moun: bool = False, num_moun_iters: int = 3,
                                                    weight_norm: bool = True):
    """lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:22-168.  Returns (o, w0, w1, w2)."""
    steps = P.ar_train_program(k.shape[1], mini_batch_size, update_length, update_every, num_repeat)
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, use_muon=use_moun, ns_steps=num_moun_iters,
                ns_const_coeffs=True, renorm=L.RENORM_EPS_OUTSIDE if weight_norm else L.RENORM_NONE,
                w_scale=w_scale, return_state=True)


def ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum(
        w0, w1, w2, q, k, v, lr0, lr1, lr2, w_scale: float, num_repeat: int = 1, mini_batch_size: int = -1,
        update_length: int = -1, update_every: int = -1, use_moun: bool = False, num_moun_iters: int = 3,
        weight_norm: bool = True, fw_momentum: torch.Tensor = None, use_momentum: bool = False):
    """lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat_sp.py:27-193 (one pass; `num_repeat`
    is accepted and ignored, as in the reference)."""
    steps = P.ar_train_program(k.shape[1], mini_batch_size, update_length, update_every, 1)
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, momentum=fw_momentum if use_momentum else None,
                use_muon=use_moun, ns_steps=num_moun_iters, ns_const_coeffs=True,
                renorm=L.RENORM_EPS_OUTSIDE if weight_norm else L.RENORM_NONE, w_scale=w_scale, return_state=True)


def ar_fast_weight_swish_glu_weight_norm_mini_batch_inference(w0, w1, w2, q, k, v, lr0, lr1, lr2, w_scale: float,
                                                              num_repeat: int = 1, mini_batch_size: int = -1,
                                                              do_update: bool = False, use_moun: bool = False,
                                                              num_moun_iters: int = 3, weight_norm: bool = True):
    """lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:171-296.  Returns (o, w0, w1, w2)."""
    steps = P.ar_inference_program(k.shape[1], mini_batch_size, do_update, num_repeat)
    return scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, use_muon=use_moun, ns_steps=num_moun_iters,
                ns_const_coeffs=True, renorm=L.RENORM_EPS_OUTSIDE if weight_norm else L.RENORM_NONE,
                w_scale=w_scale, return_state=True)


def ar_fast_weight_swish_glu_weight_norm_mini_batch_inference_with_momentum(
        w0, w1, w2, q, k, v, lr0, lr1, lr2, w_scale: float, num_repeat: int = 1, mini_batch_size: int = -1,
        do_update: bool = False, use_moun: bool = False, num_moun_iters: int = 3, weight_norm: bool = True,
        fw_momentum: torch.Tensor = None, dw0_momentum: torch.Tensor = None, dw1_momentum: torch.Tensor = None,
        dw2_momentum: torch.Tensor = None, use_momentum: bool = False):
    """lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat_sp.py:196-339.  Returns
    (o, w0, w1, w2, dw0_momentum, dw1_momentum, dw2_momentum); the momentum entries are None
    when momentum is off and none was passed in."""
    steps = P.ar_inference_program(k.shape[1], mini_batch_size, do_update, num_repeat)
    m_init = None
    if use_momentum and dw0_momentum is not None:
        m_init = (dw0_momentum, dw1_momentum, dw2_momentum)
    res = scan(w0, w1, w2, q, k, v, lr0, lr1, lr2, steps, momentum=fw_momentum if use_momentum else None,
               m_init=m_init, use_muon=use_moun, ns_steps=num_moun_iters, ns_const_coeffs=True,
               renorm=L.RENORM_EPS_OUTSIDE if weight_norm else L.RENORM_NONE, w_scale=w_scale, return_state=True,
               return_momentum=use_momentum and do_update)
    if use_momentum and do_update:
        return res
    o, a, b, c = res
    if use_momentum:  # no update ran: the state passes through (zeros if none was given)
        if dw0_momentum is None:
            dw0_momentum, dw1_momentum, dw2_momentum = (torch.zeros_like(t) for t in (a, b, c))
        return o, a, b, c, dw0_momentum, dw1_momentum, dw2_momentum
    return o, a, b, c, dw0_momentum, dw1_momentum, dw2_momentum


# ----------------------------------------------------------------------------------------------
# fused sub-ops, reference signatures
# ----------------------------------------------------------------------------------------------
def _bf16_contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != BF16:
        raise AssertionError(f"{name} must be bfloat16")  # the reference launchers assert bf16 inputs
    return t.contiguous()


# The three fused sub-ops that the reference wraps in autograd Functions (FusedSwiGLUFFNFwd, FusedLactSwiGLUFFNBwd,
# L2NormAddFunction) are registered operators with a fake implementation and an autograd formula: a caller that
# differentiates through them, or compiles them, gets what the reference's Functions give.
@torch.library.custom_op("lact_b200::swiglu_ffn_fwd", mutates_args=(), device_types="cuda")
def _swiglu_ffn_fwd_op(W0_W2: torch.Tensor, W1: torch.Tensor, X: torch.Tensor) -> torch.Tensor:
    dev = X.device
    W0_W2, W1, X = W0_W2.contiguous(), W1.contiguous(), X.contiguous()
    B, N, D = X.shape
    H = W0_W2.shape[1] // 2
    out = torch.empty(B, N, D, dtype=BF16, device=dev)
    lib = L.lib()
    need = C.c_size_t(0)
    L.check(lib.lact_swiglu_ffn_workspace_bytes(B, N, D, H, C.byref(need)), "lact_swiglu_ffn_workspace_bytes")
    ws = L.workspace(need.value, dev)
    with torch.cuda.device(dev):
        L.check(lib.lact_swiglu_ffn_fwd(W0_W2.data_ptr(), W1.data_ptr(), X.data_ptr(), out.data_ptr(), B, N, D, H,
                                        ws.data_ptr(), ws.numel(), L.stream_ptr()), "lact_swiglu_ffn_fwd")
    L.mark_pending(ws)
    return out


@_swiglu_ffn_fwd_op.register_fake
def _swiglu_ffn_fwd_fake(W0_W2, W1, X):
    return X.new_empty(X.shape)


@torch.library.custom_op("lact_b200::swiglu_ffn_bwd", mutates_args=(), device_types="cuda")
def _swiglu_ffn_bwd_op(W0_W2: torch.Tensor, W1: torch.Tensor, X: torch.Tensor,
                       grad_out: torch.Tensor) -> List[torch.Tensor]:
    """(grad_W0_W2, grad_W1, grad_X), bf16: lact_swiglu_ffn.py:46-76 (pre-activations recomputed)."""
    from .backward import apply_backward, post_status, reset_status
    reset_status(X.device)
    dW02 = torch.zeros(W0_W2.shape, dtype=torch.float32, device=X.device)
    dW1 = torch.zeros(W1.shape, dtype=torch.float32, device=X.device)
    dX = apply_backward(W0_W2.contiguous(), W1.contiguous(), X.contiguous(), grad_out.to(BF16).contiguous(), dW02, dW1)
    post_status(X.device)
    return [dW02.to(BF16), dW1.to(BF16), dX]


@_swiglu_ffn_bwd_op.register_fake
def _swiglu_ffn_bwd_fake(W0_W2, W1, X, grad_out):
    return [torch.empty_like(W0_W2), torch.empty_like(W1), torch.empty_like(X)]


def _swiglu_ffn_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _swiglu_ffn_autograd(ctx, grad_out):
    return tuple(torch.ops.lact_b200.swiglu_ffn_bwd(*ctx.saved_tensors, grad_out))


_swiglu_ffn_fwd_op.register_autograd(_swiglu_ffn_autograd, setup_context=_swiglu_ffn_setup)


def fused_swiglu_ffn_fwd(W0_W2: torch.Tensor, W1: torch.Tensor, X: torch.Tensor) -> torch.Tensor:
    """lact_llm/lact_model/lact_triton_kernels/lact_swiglu_ffn.py:79-96: W0_W2 [B, 2H, D],
    W1 [B, D, H], X [B, N, D] (bf16) -> [B, N, D].  Differentiable as FusedSwiGLUFFNFwd (:19-76) is."""
    _need_cuda(W0_W2, W1, X)
    W0_W2, W1, X = _bf16_contig(W0_W2, "W0_W2"), _bf16_contig(W1, "W1"), _bf16_contig(X, "X")
    B, N, D = X.shape
    H = W0_W2.shape[1] // 2
    assert W0_W2.shape == (B, 2 * H, D) and W1.shape == (B, D, H)
    return torch.ops.lact_b200.swiglu_ffn_fwd(W0_W2, W1, X)


@torch.library.custom_op("lact_b200::fw_grads_fwd", mutates_args=(), device_types="cuda")
def _fw_grads_fwd_op(W0_W2: torch.Tensor, W1: torch.Tensor, K: torch.Tensor, V: torch.Tensor, lr0: torch.Tensor,
                     lr1: torch.Tensor, lr2: torch.Tensor) -> List[torch.Tensor]:
    dev = K.device
    B, N, D = K.shape
    H = W0_W2.shape[1] // 2
    dw02 = torch.empty(B, 2 * H, D, dtype=BF16, device=dev)
    dw1 = torch.empty(B, D, H, dtype=BF16, device=dev)
    lib = L.lib()
    need = C.c_size_t(0)
    L.check(lib.lact_fw_grad_workspace_bytes(B, N, D, H, C.byref(need)), "lact_fw_grad_workspace_bytes")
    ws = L.workspace(need.value, dev)
    with torch.cuda.device(dev):
        L.check(lib.lact_fw_grad(W0_W2.data_ptr(), W1.data_ptr(), K.data_ptr(), V.data_ptr(), lr0.data_ptr(),
                                 lr1.data_ptr(), lr2.data_ptr(), L.dtype_code(lr0), dw02.data_ptr(), dw1.data_ptr(),
                                 B, N, D, H, ws.data_ptr(), ws.numel(), L.stream_ptr()), "lact_fw_grad")
    L.mark_pending(ws)
    return [dw02, dw1]


@_fw_grads_fwd_op.register_fake
def _fw_grads_fwd_fake(W0_W2, W1, K, V, lr0, lr1, lr2):
    return [torch.empty_like(W0_W2), torch.empty_like(W1)]


@torch.library.custom_op("lact_b200::fw_grads_bwd", mutates_args=(), device_types="cuda")
def _fw_grads_bwd_op(W0_W2: torch.Tensor, W1: torch.Tensor, K: torch.Tensor, V: torch.Tensor, lr0: torch.Tensor,
                     lr1: torch.Tensor, lr2: torch.Tensor, g02: torch.Tensor, g1: torch.Tensor) -> List[torch.Tensor]:
    """Gradients of (W0_W2, W1, K, V, lr0, lr1, lr2) given those of (DW0_DW2, DW1): the hand-written second-order
    backward of lact_fw_grad.py:61-156 (bf16 for weights and activations, fp32 row sums for the learning rates)."""
    from .backward import fw_grad_backward, post_status, reset_status
    reset_status(K.device)
    dW02 = torch.zeros(W0_W2.shape, dtype=torch.float32, device=K.device)
    dW1 = torch.zeros(W1.shape, dtype=torch.float32, device=K.device)
    dk, dv, g0, g1_, g2 = fw_grad_backward(W0_W2, W1, K, V, lr0, lr1, lr2, 1.0, g02, g1, dW02, dW1)
    post_status(K.device)
    return [dW02.to(BF16), dW1.to(BF16), dk, dv, g0.to(lr0.dtype), g1_.to(lr1.dtype), g2.to(lr2.dtype)]


@_fw_grads_bwd_op.register_fake
def _fw_grads_bwd_fake(W0_W2, W1, K, V, lr0, lr1, lr2, g02, g1):
    return [torch.empty_like(t) for t in (W0_W2, W1, K, V, lr0, lr1, lr2)]


def _fw_grads_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)
    ctx.set_materialize_grads(False)


def _fw_grads_autograd(ctx, grads):
    W0_W2, W1 = ctx.saved_tensors[:2]
    g02 = grads[0] if grads[0] is not None else torch.zeros_like(W0_W2)
    g1 = grads[1] if grads[1] is not None else torch.zeros_like(W1)
    return tuple(torch.ops.lact_b200.fw_grads_bwd(*ctx.saved_tensors, g02.contiguous(), g1.contiguous()))


_fw_grads_fwd_op.register_autograd(_fw_grads_autograd, setup_context=_fw_grads_setup)


def fused_lact_swiglu_ffn_fast_weight_grads(W0_W2, W1, K, V, lr0, lr1, lr2):
    """lact_llm/lact_model/lact_triton_kernels/lact_fw_grad.py:159-175: returns (DW0_DW2
    [B, 2H, D], DW1 [B, D, H]) in bf16; lr0/1/2 are [B, N].  Differentiable as FusedLactSwiGLUFFNBwd (:21-156) is."""
    _need_cuda(W0_W2, W1, K, V, lr0, lr1, lr2)
    W0_W2, W1 = _bf16_contig(W0_W2, "W0_W2"), _bf16_contig(W1, "W1")
    K, V = _bf16_contig(K, "K"), _bf16_contig(V, "V")
    B, N, D = K.shape
    lr0, lr1, lr2 = (_vec(t, B, N, "lr") for t in (lr0, lr1, lr2))
    if not (lr0.dtype == lr1.dtype == lr2.dtype):
        lr0, lr1, lr2 = lr0.float(), lr1.float(), lr2.float()
    dw02, dw1 = torch.ops.lact_b200.fw_grads_fwd(W0_W2, W1, K, V, lr0, lr1, lr2)
    return dw02, dw1


def l2_norm(x: torch.Tensor) -> torch.Tensor:
    """x scaled to unit l2 norm along its last axis, `x / (||x|| + 1e-5)` with the norm, the sum and the quotient each
    in x's dtype (lact_llm/lact_model/ttt_operation.py:19-26; the layer imports it next to the chunk drivers,
    layer_lact_swiglu.py:20-24).  Plain tensor arithmetic, exported so that the layer's import line keeps working; the
    fused pass over q, k, v (`layer_ops.qkv_prologue`: head split, SiLU and this normalisation in one kernel) is what
    a layer on this package calls instead."""
    return (x / (x.norm(dim=-1, keepdim=True) + 1e-5)).type(x.dtype)


class _NewtonSchulz(torch.autograd.Function):
    """U = NS(G) with every iterate kept (`lact_ns_trace_fwd`); dG from `lact_ns_trace_bwd` (bf16 operands, roundings
    treated as identities, as autograd through the reference's bf16 iteration does) and the Frobenius normalisation."""
    @staticmethod
    def forward(ctx, G, steps):
        from .backward import ns_forward_saved
        Gd = G.detach()
        ctx.saved, U = ns_forward_saved(Gd, 5 if steps is None else int(steps), steps is not None, False)
        ctx.in_dtype = G.dtype
        return U

    @staticmethod
    def backward(ctx, dU):
        from .backward import ns_backward, post_status
        dG = ns_backward(ctx.saved, dU.contiguous())
        post_status(dG.device)
        return dG.to(ctx.in_dtype), None


@_no_trace
def zeropower_via_newtonschulz5(G: torch.Tensor, steps: Optional[int] = None) -> torch.Tensor:
    """Newton-Schulz orthogonalisation in bf16.  `steps=None`: the tuned 5-step schedule of
    lact_llm/lact_model/ttt_operation.py:30-66; `steps=int`: the constant-coefficient variant of
    lact_nvs/lact_ttt.py:32-67.  G: [b, r, c], any float dtype -> bf16 [b, r, c]."""
    assert len(G.shape) == 3
    dev = _need_cuda(G)
    if torch.is_grad_enabled() and G.requires_grad:
        # the reference's function is plain PyTorch and so differentiable: here the iterates are kept and walked
        # backwards by the recurrence's own Newton-Schulz backward kernels
        return _NewtonSchulz.apply(G, steps)
    if G.dtype not in (torch.float32, BF16):
        G = G.float()
    G = G.contiguous()
    B, R, Cc = G.shape
    x = torch.empty(B, R, Cc, dtype=BF16, device=dev)
    lib = L.lib()
    need = C.c_size_t(0)
    L.check(lib.lact_newton_schulz_workspace_bytes(B, R, Cc, C.byref(need)), "lact_newton_schulz_workspace_bytes")
    ws = L.workspace(need.value, dev)
    with torch.cuda.device(dev):
        L.check(lib.lact_newton_schulz(G.data_ptr(), L.dtype_code(G), x.data_ptr(), B, R, Cc,
                                       5 if steps is None else int(steps), int(steps is not None), ws.data_ptr(),
                                       ws.numel(), L.stream_ptr()), "lact_newton_schulz")
    L.mark_pending(ws)
    return x


@torch.library.custom_op("lact_b200::l2_norm_add_fwd", mutates_args=(), device_types="cuda")
def _l2_norm_add_fwd_op(x: torch.Tensor, x_add: torch.Tensor, tgt_scale: torch.Tensor, eps: float,
                        out_bf16: bool) -> torch.Tensor:
    dev = x.device
    x, x_add = x.contiguous(), x_add.contiguous()
    B, T, D = x.shape
    sc = tgt_scale.reshape(B, T).float().contiguous()
    y = torch.empty(B, T, D, dtype=BF16 if out_bf16 else torch.float32, device=dev)
    with torch.cuda.device(dev):
        L.check(L.lib().lact_l2_norm_add(x.data_ptr(), L.dtype_code(x), x_add.data_ptr(), L.dtype_code(x_add),
                                         sc.data_ptr(), y.data_ptr(), L.dtype_code(y), B, T, D, float(eps),
                                         L.stream_ptr()), "lact_l2_norm_add")
    return y


@_l2_norm_add_fwd_op.register_fake
def _l2_norm_add_fwd_fake(x, x_add, tgt_scale, eps, out_bf16):
    return x.new_empty(x.shape, dtype=BF16 if out_bf16 else torch.float32)


@torch.library.custom_op("lact_b200::l2_norm_add_bwd", mutates_args=(), device_types="cuda")
def _l2_norm_add_bwd_op(x: torch.Tensor, x_add: torch.Tensor, tgt_scale: torch.Tensor, dy: torch.Tensor,
                        eps: float) -> List[torch.Tensor]:
    """(dx, dx_add, dtgt_scale) of y = (x + x_add) * rsqrt(sum (x + x_add)^2 + eps) * tgt_scale
    (l2norm_triton_kernels.py:97-172, 409-416); the row is recomputed from the inputs."""
    from .backward import renorm_backward
    if abs(float(eps) - 1e-5) > 1e-12:
        raise NotImplementedError("the backward of l2_norm_add_fused is built for eps = 1e-5 (the value every caller uses)")
    B, T, D = x.shape
    sc = tgt_scale.reshape(B, T).float().contiguous()
    dsc = torch.zeros(B, T, dtype=torch.float32, device=x.device)
    dw = renorm_backward(x.float().contiguous(), x_add, sc, dy.float().contiguous(), dsc, L.RENORM_EPS_INSIDE)
    # (two distinct tensors even where both inputs have dw's dtype: an operator's outputs may not alias one another)
    dxa = dw.to(x_add.dtype) if x_add.dtype != dw.dtype else dw.clone()
    return [dw.to(x.dtype), dxa, dsc.reshape(tgt_scale.shape).to(tgt_scale.dtype)]


@_l2_norm_add_bwd_op.register_fake
def _l2_norm_add_bwd_fake(x, x_add, tgt_scale, dy, eps):
    return [torch.empty_like(x), torch.empty_like(x_add), torch.empty_like(tgt_scale)]


def _l2_norm_add_setup(ctx, inputs, output):
    x, x_add, tgt_scale, eps, _ = inputs
    ctx.save_for_backward(x, x_add, tgt_scale)
    ctx.eps = float(eps)


def _l2_norm_add_autograd(ctx, dy):
    x, x_add, tgt_scale = ctx.saved_tensors
    dx, dxa, dsc = torch.ops.lact_b200.l2_norm_add_bwd(x, x_add, tgt_scale, dy.contiguous(), ctx.eps)
    return dx, dxa, dsc, None, None


_l2_norm_add_fwd_op.register_autograd(_l2_norm_add_autograd, setup_context=_l2_norm_add_setup)


def l2_norm_add_fused(x, x_add, tgt_scale, eps: float = 1e-5, tgt_dtype=None) -> torch.Tensor:
    """lact_llm/lact_model/lact_triton_kernels/l2norm_triton_kernels.py:419-427.  Differentiable as
    L2NormAddFunction (:386-416) is."""
    _need_cuda(x, x_add, tgt_scale)
    tgt_dtype = x.dtype if tgt_dtype is None else tgt_dtype
    if tgt_dtype not in (torch.float32, BF16):
        raise TypeError("tgt_dtype must be float32 or bfloat16")
    if x.dtype not in (torch.float32, BF16):
        x = x.float()
    if x_add.dtype not in (torch.float32, BF16):
        x_add = x_add.float()
    return torch.ops.lact_b200.l2_norm_add_fwd(x, x_add, tgt_scale, float(eps), tgt_dtype == BF16)


@_no_trace
def fused_prenorm_update_with_momentum_and_l2_norm(x_main, dx, dx_momentum, momentum_mu, tgt_scale, eps: float = 1e-5):
    """lact_llm/lact_model/lact_triton_kernels/triton_prenorm_update_with_momentum.py:379-401.
    Returns (y_main fp32, updated_momentum fp32, y_normalized bf16)."""
    dev = _need_cuda(x_main, dx, dx_momentum, momentum_mu, tgt_scale)
    B, T, D = x_main.shape
    x = x_main.float().contiguous()
    m = dx_momentum.float().contiguous()
    dxb = dx.to(BF16).contiguous()
    mu = momentum_mu.float().contiguous()
    sc = tgt_scale.float().contiguous()
    xo, mo = torch.empty_like(x), torch.empty_like(m)
    yo = torch.empty(B, T, D, dtype=BF16, device=dev)
    with torch.cuda.device(dev):
        L.check(L.lib().lact_prenorm_momentum_l2norm(x.data_ptr(), dxb.data_ptr(), m.data_ptr(), mu.data_ptr(),
                                                     sc.data_ptr(), xo.data_ptr(), mo.data_ptr(), yo.data_ptr(), B, T,
                                                     D, float(eps), L.stream_ptr()), "lact_prenorm_momentum_l2norm")
    return xo, mo, yo


@_no_trace
def bmm_bf16(a: torch.Tensor, b: torch.Tensor, a_mn_major: bool = False, b_mn_major: bool = False,
             out_dtype=torch.float32) -> torch.Tensor:
    """c = A B^T on the tcgen05 engine (test hook).  a: [batch, M, K] or, MN-major, [batch, K, M];
    b: [batch, N, K] or [batch, K, N]."""
    dev = _need_cuda(a, b)
    a, b = _bf16_contig(a, "a"), _bf16_contig(b, "b")
    batch = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mn_major else (a.shape[1], a.shape[2])
    N = b.shape[2] if b_mn_major else b.shape[1]
    c = torch.empty(batch, M, N, dtype=out_dtype, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        L.check(L.lib().lact_bmm_bf16(a.data_ptr(), int(a_mn_major), b.data_ptr(), int(b_mn_major), c.data_ptr(),
                                      L.dtype_code(c), batch, M, N, K, status.data_ptr(), L.stream_ptr()),
                "lact_bmm_bf16")
    st = int(status[0].item())
    if st != 0:
        raise L.LactError(f"device status {st}")
    return c
