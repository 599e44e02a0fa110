"""Data parallelism over sequences: the only parallel strategy on this path.

The reference accumulates gradients one example at a time with a global per-target weight
1/batch_tokens (src/train.rs:263,275,330), so a batch is a sum over independent sequences.
Ranks take sequences round-robin, compute their partial LoRA gradients with the GLOBAL weight,
and one all-reduce (sum) of the flat gradient buffer per step makes every rank's gradient the
full-batch one; each rank then runs the identical clip + AdamW, so parameters stay equal without
a broadcast.

`local_batch` is the host-side rule (which sequences, which targets, which weights); the exchange
itself is whatever the caller passes: on GPUs the library's own NCCL communicator
(`Model.allreduce_grads`, rt_comm_* in the C ABI), in the CPU tests a gloo all-reduce.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .synth import answer_targets


def shard_sequences(n_seq: int, rank: int, world: int) -> list:
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return list(range(rank, n_seq, world))


def global_batch_tokens(answer_lens: list) -> int:
    """Sum of answer lengths over the WHOLE batch (src/train.rs:330), at least 1."""
    return max(int(sum(answer_lens)), 1)


@dataclass
class LocalBatch:
    seqs: list               # this rank's sequences (int32 arrays), in global order
    indices: list            # their indices in the global batch
    target_pos: np.ndarray   # positions in the concatenation of `seqs`
    target_tok: np.ndarray
    weights: np.ndarray      # 1 / global batch_tokens on every target
    per_seq: list            # (target_pos within the sequence, target_tok) per local sequence
    batch_tokens: int        # the GLOBAL number of answer tokens


def local_batch(examples, rank: int, world: int) -> LocalBatch:
    """examples: the GLOBAL batch as [(tokens, answer_start)].  Every rank calls this with the same
    list and gets its round-robin share, weighted so that the ranks' gradients SUM to the batch
    gradient (src/train.rs:330: batch_tokens is counted over the whole batch)."""
    lens = []
    for toks, a0 in examples:
        lens.append(max(int(np.asarray(toks).size) - max(int(a0), 1), 0))
    bt = global_batch_tokens(lens)
    idx = shard_sequences(len(examples), rank, world)
    seqs, tps, tts, per_seq, off = [], [], [], [], 0
    for i in idx:
        toks = np.ascontiguousarray(examples[i][0], dtype=np.int32)
        tp, tt = answer_targets(toks, examples[i][1])
        seqs.append(toks)
        per_seq.append((tp, tt))
        tps.append(tp + off)
        tts.append(tt)
        off += toks.size
    cat = lambda parts, dt: np.concatenate(parts).astype(dt) if parts else np.zeros(0, dt)
    tp, tt = cat(tps, np.int32), cat(tts, np.int32)
    return LocalBatch(seqs, idx, tp, tt, np.full(tp.size, 1.0 / bt, np.float32), per_seq, bt)


def step_loss(logp: np.ndarray, batch: LocalBatch) -> float:
    """This rank's share of the step loss -sum(logp)/batch_tokens (src/train.rs:365); the shares
    add up over ranks."""
    return float(-np.sum(logp.astype(np.float64)) / batch.batch_tokens)


def allreduce_sum_(tensor, group=None):
    """In-place sum over ranks of a torch tensor (CPU tests: gloo)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
    return tensor
