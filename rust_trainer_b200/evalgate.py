"""Forward-only scoring for the eval gate (reference src/eval.rs:156-221) on the device model:
`greedy_prefix`, `greedy_prefix_batch` and the packing rule `worth_packing`, which the trainer
consults too (src/train.rs:255)."""
from __future__ import annotations

import os

import numpy as np

from .packing import Packed, pack


def worth_packing(seqs) -> Packed | None:
    """Pack a batch only when the shared prompt is at least half of an average example
    (src/eval.rs:176-186); `RT_NO_PACK` set turns packing off.  Every model this library builds
    supports packing (dense attention layers only)."""
    if len(seqs) < 2 or os.environ.get("RT_NO_PACK") is not None:
        return None
    p = pack(seqs)
    avg = sum(int(np.asarray(s).size) for s in seqs) // len(seqs)
    return p if p.shared * 2 >= avg else None


def _prefix_len(argmax: np.ndarray, want: np.ndarray) -> int:
    ok = 0
    for a, w in zip(argmax.tolist(), want.tolist()):
        if a != w:
            break
        ok += 1
    return ok


def greedy_prefix(model, tokens, answer_start: int):
    """(length of the answer prefix greedy decoding reproduces, answer length): the argmax is
    right at every answer position under teacher forcing iff greedy decoding emits the whole
    answer (src/eval.rs:152-173)."""
    tokens = np.asarray(tokens, dtype=np.int32)
    start = max(int(answer_start), 1)
    if start >= tokens.size:
        return 0, 0
    pos = np.arange(start - 1, tokens.size - 1, dtype=np.int32)
    am = model.argmax_at([tokens], pos)
    return _prefix_len(am, tokens[start:]), pos.size


def greedy_prefix_batch(model, examples):
    """`greedy_prefix` of several (tokens, answer_start) examples, sharing their common prompt when
    `worth_packing` says so (src/eval.rs:189-221); otherwise one batched pass over the examples."""
    exs = [(np.asarray(t, dtype=np.int32), max(int(a), 1)) for t, a in examples]
    if not exs:
        return []
    p = worth_packing([t for t, _ in exs])
    all_pos, spans, off = [], [], 0
    for k, (t, start) in enumerate(exs):
        lo = len(all_pos)
        for q in range(start - 1, max(t.size - 1, 0)):
            all_pos.append(p.index(k, q) if p is not None else off + q)
        spans.append((lo, len(all_pos), start))
        off += t.size
    if not all_pos:
        return [(0, 0) for _ in exs]
    pos = np.asarray(all_pos, dtype=np.int32)
    am = model.argmax_at_packed([p], pos) if p is not None else model.argmax_at([t for t, _ in exs], pos)
    return [(_prefix_len(am[a:b], t[start:start + (b - a)]), b - a) for (t, start), (a, b, _) in zip(exs, spans)]
