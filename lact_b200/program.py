"""Step programs: the index arithmetic of every reference chunk driver, as plain integers.

A program is a list of (kind, start, end, out_start) with kind APPLY or UPDATE; APPLY writes
o[:, out_start : out_start + end - start] from q[:, start:end] with the current fast weights,
UPDATE updates the fast weights from k, v, lr on [start, end).  Slices follow Python's clamping
rules, as in the reference.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

APPLY = 0
UPDATE = 1
Step = Tuple[int, int, int, int]


def causal_program(L: int, chunk_size: int) -> List[Step]:
    """Apply-then-update per chunk, last chunk apply only.

    lact_llm/lact_model/ttt_operation.py:124-212 (`range(0, seq_len - chunk_size, chunk_size)`,
    tail `[e_index, seq_len)`).  The fused functions pad to a chunk multiple and update on all
    but the last chunk (ttt_operation_fused_kernel.py:112-182); after truncating the padding this
    is the same list of token ranges.
    """
    if chunk_size < 1:
        raise ValueError("chunk_size must be positive")
    steps: List[Step] = []
    e = 0
    for s in range(0, L - chunk_size, chunk_size):
        e = s + chunk_size
        steps.append((APPLY, s, e, s))
        steps.append((UPDATE, s, e, 0))
    steps.append((APPLY, e, L, e))
    return steps


def bidirectional_program(L: int) -> List[Step]:
    """One update on every token, then apply to every token.
    minimal_implementations/bidirectional_lact_layer.py:116-158."""
    return [(UPDATE, 0, L, 0), (APPLY, 0, L, 0)]


def _clamp(start: int, end: int, L: int) -> Tuple[int, int]:
    s = max(0, min(L, start if start >= 0 else L + start))
    e = max(0, min(L, end if end >= 0 else L + end))
    return s, max(s, e)


def operator_list_program(order: Sequence[Sequence], L: int) -> Tuple[List[Step], int]:
    """(start, end, update, apply) operators; apply outputs are concatenated in list order.
    lact_nvs/lact_ttt.py:100-145.  Returns (steps, total output length)."""
    steps: List[Step] = []
    out = 0
    for start, end, update, apply in order:
        s, e = _clamp(int(start), int(end), L)
        if update:
            steps.append((UPDATE, s, e, 0))
        if apply:
            steps.append((APPLY, s, e, out))
            out += e - s
    return steps, out


def ar_train_program(L: int, mini_batch_size: int = -1, update_length: int = -1, update_every: int = -1,
                     num_repeat: int = 1) -> List[Step]:
    """Apply the first `update_every - mini_batch_size` tokens with the initial weights, then for
    every stride: update on `mini_batch_size` tokens, apply on `update_every` tokens.
    lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:74-165."""
    if update_length == -1:
        update_length = L
    if mini_batch_size == -1:
        mini_batch_size = update_length
    if update_every == -1:
        update_every = mini_batch_size * 2
    if update_every < 1:
        raise ValueError("update_every must be positive")
    first = update_every - mini_batch_size
    steps: List[Step] = []
    s0, e0 = _clamp(0, first, L)
    steps.append((APPLY, s0, e0, s0))
    for _ in range(num_repeat):
        for s in range(first, update_length, update_every):
            us, ue = _clamp(s, s + mini_batch_size, L)
            steps.append((UPDATE, us, ue, 0))
            a_s, a_e = _clamp(s, s + update_every, L)
            steps.append((APPLY, a_s, a_e, a_s))
    return steps


def ar_inference_program(L: int, mini_batch_size: int = -1, do_update: bool = False, num_repeat: int = 1) -> List[Step]:
    """Optional `num_repeat` updates on the first mini-batch, then apply to every token.
    lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:231-293."""
    if mini_batch_size == -1:
        mini_batch_size = L
    steps: List[Step] = []
    if do_update:
        for _ in range(num_repeat):
            us, ue = _clamp(0, mini_batch_size, L)
            steps.append((UPDATE, us, ue, 0))
    steps.append((APPLY, 0, L, 0))
    return steps


import collections  # noqa: E402

# Same field names as the reference's operator tuple (lact_nvs/lact_ttt.py:10).
TTTOperator = collections.namedtuple("TTTOperator", ["start", "end", "update", "apply"])
