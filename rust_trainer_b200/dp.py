"""Data parallelism over sequences: the only parallel strategy on this path.

The reference accumulates gradients one example at a time with a global per-target weight
1/batch_tokens (src/train.rs:263,275,330), so a batch is a sum over independent sequences.
Ranks take sequences round-robin, compute their partial LoRA gradients with the GLOBAL
weight, and one all-reduce (sum) of the flat gradient buffer per step makes every rank's
gradient the full-batch one; each rank then runs the identical clip + AdamW, so parameters
stay equal without a broadcast.  torch.distributed is plumbing only (NCCL on GPUs, gloo in
the CPU tests).
"""
from __future__ import annotations


def shard_sequences(n_seq: int, rank: int, world: int) -> list:
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return list(range(rank, n_seq, world))


def global_batch_tokens(answer_lens: list) -> int:
    """Sum of answer lengths over the WHOLE batch (src/train.rs:330), at least 1."""
    return max(int(sum(answer_lens)), 1)


def allreduce_sum_(tensor, group=None):
    """In-place sum over ranks of a torch tensor (the flat LoRA-gradient buffer or the loss)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
    return tensor
