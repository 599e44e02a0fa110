"""Shared-prompt packing (reference src/model.rs:234-290).

Several examples that start with the same prompt are laid out as one sequence
`[shared prompt | rest of example 0 | rest of example 1 | ...]`; every token keeps its position
within its own example (RoPE) and attends to the shared prompt and to its own example's earlier
tokens only.  The result equals running the examples separately, while the prompt is computed,
forward and backward, once.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class Packed:
    tokens: np.ndarray     # int32
    positions: np.ndarray  # int32, position of each token within its own example
    segments: np.ndarray   # int32, 0 = shared prompt, k + 1 = example k
    shared: int            # length of the shared prompt
    offsets: list          # where each example's own tokens start in `tokens`

    def index(self, k: int, pos: int) -> int:
        """Index in `tokens` of position `pos` of example `k` (Packed::index)."""
        return pos if pos < self.shared else self.offsets[k] + pos - self.shared

    def map_targets(self, k: int, target_pos, target_tok):
        """Example k's targets (as for its own sequence) mapped into the packed sequence."""
        tp = np.array([self.index(k, int(p)) for p in np.asarray(target_pos)], dtype=np.int32)
        return tp, np.asarray(target_tok, dtype=np.int32)


def pack(seqs) -> Packed:
    """The shared part is the longest common prefix, kept short enough that every sequence has at
    least one token of its own; a single sequence shares nothing (src/model.rs:266-290)."""
    seqs = [np.asarray(s, dtype=np.int32) for s in seqs]
    assert seqs, "nothing to pack"
    min_len = min(s.size for s in seqs)
    shared = 0
    while shared + 1 < min_len and all(s[shared] == seqs[0][shared] for s in seqs):
        shared += 1
    if len(seqs) == 1:
        shared = 0
    toks, pos, seg, offsets = [seqs[0][:shared]], [np.arange(shared, dtype=np.int32)], [np.zeros(shared, np.int32)], []
    n = shared
    for k, s in enumerate(seqs):
        offsets.append(n)
        toks.append(s[shared:])
        pos.append(np.arange(shared, s.size, dtype=np.int32))
        seg.append(np.full(s.size - shared, k + 1, np.int32))
        n += s.size - shared
    return Packed(np.concatenate(toks).astype(np.int32), np.concatenate(pos), np.concatenate(seg), shared, offsets)
