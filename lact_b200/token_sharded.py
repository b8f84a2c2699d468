"""Token-sharded fast-weight recurrence (context parallel inside a chunk) for shapes with few
(batch x head) entries: the entries cannot fill several GPUs, the tokens of a chunk can.

Every rank holds the same fast weights and 1/W of every chunk's tokens.  Apply is token-local.  The
fast-weight gradient is a sum over the chunk's tokens, so each rank contracts its own tokens and the
partial gradients (and the partial sums of the momentum gate) are added across ranks in ONE
all-reduce per chunk over NCCL / NVLink; momentum, Newton-Schulz and the renormalisation are then
replicated, so the weights stay bit-identical on all ranks without ever being broadcast.  The
reference has no such driver; the recurrence is that of its fused post-norm function
(lact_llm/lact_model/ttt_operation_fused_kernel.py:66-186) and the sharding pattern follows its
sequence-parallel helpers (lact_ar_video/minVid/models/wan/wan_base/distributed/sp_support.py:65-144).

Token layout: with chunk size C and W ranks, rank r holds tokens [r * C/W, (r+1) * C/W) of every
chunk, chunks concatenated in order (`shard_tokens` / `unshard_tokens`).

Training: the recurrence is built from the differentiable sub-ops (the Newton-Schulz one included), and the all-reduce
is an autograd node whose backward all-reduces the incoming gradient (every rank's loss depends on the summed
gradient).  Each rank gets the gradients of its own token shards (q, k, v, learning rates, momentum) in full; the
gradients of the REPLICATED initial weights come out as per-rank shares that the caller sums over the ranks, as a
data-parallel wrapper does for any replicated parameter.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

BF16 = torch.bfloat16


def shard_tokens(x: torch.Tensor, chunk_size: int, world_size: int, rank: int) -> torch.Tensor:
    """[B, L, ...] -> this rank's [B, L / W, ...]: its 1/W slice of every chunk.  L must be a multiple of the
    chunk size and the chunk size a multiple of W."""
    B, L = x.shape[:2]
    if L % chunk_size or chunk_size % world_size:
        raise ValueError("token sharding needs L % chunk_size == 0 and chunk_size % world_size == 0")
    per = chunk_size // world_size
    xs = x.reshape(B, L // chunk_size, world_size, per, *x.shape[2:])
    return xs[:, :, rank].reshape(B, (L // chunk_size) * per, *x.shape[2:]).contiguous()


def unshard_tokens(parts: List[torch.Tensor], chunk_size: int) -> torch.Tensor:
    """Inverse of `shard_tokens` given the shards of all ranks in rank order."""
    W = len(parts)
    per = chunk_size // W
    B, Lloc = parts[0].shape[:2]
    n_chunks = Lloc // per
    st = torch.stack([p.reshape(B, n_chunks, per, *p.shape[2:]) for p in parts], dim=2)
    return st.reshape(B, n_chunks * chunk_size, *parts[0].shape[2:])


class _AllReduceSum(torch.autograd.Function):
    """y = sum over ranks of x (every rank receives y); dL/dx = sum over ranks of dL/dy."""
    @staticmethod
    def forward(ctx, x, all_reduce):
        ctx.all_reduce = all_reduce
        y = x.detach().clone()
        all_reduce(y)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        ctx.all_reduce(g)
        return g, None


def _cuda_ops() -> SimpleNamespace:
    """The library's fused sub-ops (CUDA); the only implementation the product uses."""
    from . import ops
    return SimpleNamespace(apply=ops.fused_swiglu_ffn_fwd, grads=ops.fused_lact_swiglu_ffn_fast_weight_grads,
                           newton_schulz=ops.zeropower_via_newtonschulz5, l2_norm_add=ops.l2_norm_add_fused)


class TokenShardedScan:
    """One rank's side of the recurrence, split at the point where ranks exchange data, so that the exchange can be
    a process-group all-reduce (`token_sharded_block_causal_lact_swiglu`) or, for tests on one device, a plain sum
    over several instances driven in lock step."""

    def __init__(self, w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size: int, world_size: int, use_muon: bool = False,
                 momentum: Optional[torch.Tensor] = None, sub_ops: Optional[SimpleNamespace] = None):
        if chunk_size % world_size:
            raise ValueError("chunk_size must be a multiple of the number of ranks")
        self.ops = sub_ops if sub_ops is not None else _cuda_ops()
        self.per = chunk_size // world_size   # tokens of one chunk on this rank
        self.chunk = chunk_size
        B, Lloc, D = q.shape
        if Lloc % self.per:
            raise ValueError("the local sequence must hold 1 / world_size of whole chunks")
        self.n_chunks = Lloc // self.per
        self.q, self.k, self.v = q, k, v
        vec = lambda t: (t[..., 0] if t.dim() == 3 else t)
        self.lr = [vec(lr0), vec(lr1), vec(lr2)]
        self.mom = vec(momentum).float() if momentum is not None else None
        self.use_muon = use_muon
        self.w02 = torch.cat([w0, w2], dim=1).float().contiguous()
        self.w1 = w1.float().contiguous()
        self.n02 = self.w02.norm(dim=2)
        self.n1 = self.w1.norm(dim=2)
        self.m02 = torch.zeros_like(self.w02) if momentum is not None else None
        self.m1 = torch.zeros_like(self.w1) if momentum is not None else None
        self.out = torch.empty_like(q)
        self.n02_el, self.n1_el = self.w02.numel(), self.w1.numel()

    def _range(self, c: int):
        return c * self.per, (c + 1) * self.per

    def apply(self, c: int) -> None:
        """o = f_W(q) on this rank's tokens of chunk c (token-local)."""
        s, e = self._range(c)
        self.out[:, s:e] = self.ops.apply(self.w02.to(BF16), self.w1.to(BF16), self.q[:, s:e].contiguous())

    def local_gradient(self, c: int) -> torch.Tensor:
        """Flat fp32 buffer [dW02 | dW1 | sum of the momentum gate] of this rank's tokens of chunk c: the summand of
        the chunk's all-reduce."""
        s, e = self._range(c)
        d02, d1 = self.ops.grads(self.w02.to(BF16), self.w1.to(BF16), self.k[:, s:e].contiguous(),
                                 self.v[:, s:e].contiguous(), *[l[:, s:e].contiguous() for l in self.lr])
        B = self.w02.shape[0]
        flat = torch.empty(self.n02_el + self.n1_el + B, dtype=torch.float32, device=self.w02.device)
        flat[:self.n02_el] = d02.reshape(-1)
        flat[self.n02_el:self.n02_el + self.n1_el] = d1.reshape(-1)
        flat[self.n02_el + self.n1_el:] = self.mom[:, s:e].sum(dim=1) if self.mom is not None else 0.0
        return flat

    def update(self, reduced: torch.Tensor) -> None:
        """Momentum, Newton-Schulz, add and renormalise from the chunk's summed gradient (identical on all ranks)."""
        dw02 = reduced[:self.n02_el].view_as(self.w02)
        dw1 = reduced[self.n02_el:self.n02_el + self.n1_el].view_as(self.w1)
        if self.mom is not None:
            beta = (reduced[self.n02_el + self.n1_el:] / float(self.chunk)).view(-1, 1, 1)
            dw02 = dw02 + self.m02 * beta
            dw1 = dw1 + self.m1 * beta
            self.m02, self.m1 = dw02, dw1
        if self.use_muon:
            dw1 = self.ops.newton_schulz(dw1)
            dw02 = self.ops.newton_schulz(dw02)
        self.w02 = self.ops.l2_norm_add(self.w02, dw02.contiguous(), self.n02, eps=1e-5)
        self.w1 = self.ops.l2_norm_add(self.w1, dw1.contiguous(), self.n1, eps=1e-5)

    def run(self, all_reduce: Callable[[torch.Tensor], None]) -> torch.Tensor:
        """Apply-then-update over the chunks; `all_reduce(t)` sums `t` in place over the ranks."""
        for c in range(self.n_chunks - 1):
            self.apply(c)
            flat = self.local_gradient(c)
            if flat.requires_grad:
                flat = _AllReduceSum.apply(flat, all_reduce)
            else:
                all_reduce(flat)
            self.update(flat)
        self.apply(self.n_chunks - 1)
        return self.out


def token_sharded_block_causal_lact_swiglu(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size: int = 2048,
                                           use_muon: bool = False, momentum: Optional[torch.Tensor] = None,
                                           group: Optional[dist.ProcessGroup] = None,
                                           sub_ops: Optional[SimpleNamespace] = None) -> torch.Tensor:
    """`postnorm_block_causal_lact_swiglu_fused_kernel_triton` with every chunk's tokens spread over the ranks of
    `group`.  q, k, v, lr*, momentum are this rank's token shards (`shard_tokens` layout), the weights are the full
    (replicated) initial fast weights; returns this rank's shard of the output.  `chunk_size` is the GLOBAL chunk
    size.  One all-reduce of [B (2HD + DH) + B] fp32 values per update; without an initialised process group the
    call degenerates to the single-rank recurrence.  Differentiable (module docstring: the weights' gradients are
    per-rank shares to be summed over the ranks)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    scan = TokenShardedScan(w0, w1, w2, q, k, v, lr0, lr1, lr2, chunk_size, world, use_muon=use_muon,
                            momentum=momentum, sub_ops=sub_ops)
    if world == 1:
        return scan.run(lambda t: None)
    return scan.run(lambda t: dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group))
