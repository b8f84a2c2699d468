"""Multi-GPU layout of the TTT step: every merged (batch x head) entry is an independent
recurrence (the reference batches all ops over dim 0 with no cross-batch term, and merges heads
into the batch before the call, lact_llm/lact_model/layer_lact_swiglu.py:399-401), so ranks own
contiguous blocks of that axis and exchange nothing during the op.  The only collective is the
optional final gather of the output.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def partition(n_entries: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[start, end) of the (batch x head) entries owned by `rank`: contiguous blocks, the first
    `n_entries % world_size` ranks hold one entry more."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world_size")
    base, extra = divmod(n_entries, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard(tensors: dict, n_entries: int, world_size: int, rank: int) -> dict:
    """Slices dim 0 of every tensor whose dim 0 equals `n_entries`."""
    s, e = partition(n_entries, world_size, rank)
    return {k: (v[s:e] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == n_entries else v)
            for k, v in tensors.items()}


def gather_output(o_local: torch.Tensor, n_entries: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers the per-rank outputs along dim 0 into [n_entries, ...] on every rank.  Blocks of
    unequal size are padded to the largest block for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    sizes = [partition(n_entries, world, r) for r in range(world)]
    biggest = max(e - s for s, e in sizes)
    padded = o_local
    if o_local.shape[0] < biggest:
        pad = torch.zeros((biggest - o_local.shape[0],) + tuple(o_local.shape[1:]), dtype=o_local.dtype,
                          device=o_local.device)
        padded = torch.cat([o_local, pad], dim=0)
    parts: List[torch.Tensor] = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[: e - s] for p, (s, e) in zip(parts, sizes)], dim=0)
