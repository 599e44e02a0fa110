"""Data-parallel step on CPU ranks (gloo, world_size 2): `dp.local_batch` shards one global batch
round-robin with the global 1/batch_tokens weight, one all-reduce sums the flat gradient buffer,
and the result equals one rank computing the whole batch.  The compute engine here is the CPU
oracle and the exchange is gloo; on GPUs the same `dp.local_batch` feeds the device model and the
exchange is the library's NCCL communicator (bench.py prints that comparison as `dp_check`)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _examples(spec):
    from rust_trainer_b200 import synth

    lens = [12, 9, 12, 7, 11]  # ragged: the ranks own different numbers of answer tokens
    toks = synth.token_batch(spec, len(lens), max(lens), 4)
    return [(toks[i][:n], 5) for i, n in enumerate(lens)]


def _grads(examples, rank, world):
    from oracle import oracle as O
    from rust_trainer_b200 import dp, synth

    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=1)
    m = O.OracleModel(spec.config(), synth.build_tensors(spec))
    m.attach_lora(synth.lora_adapters(spec, 4, 8.0, 2, b_std=0.02))
    b = dp.local_batch(examples, rank, world)
    m.zero_grad()
    loss, k = 0.0, 0
    for s, (tp, tt) in zip(b.seqs, b.per_seq):
        lp, _ = m.forward_backward(s, tp, tt, b.weights[k:k + tp.size])
        loss += -float(lp.astype(np.float64).sum()) / b.batch_tokens
        k += tp.size
    flat = np.concatenate([np.concatenate([e["ga"].ravel(), e["gb"].ravel()]) for e in m.lora])
    return flat, loss, b


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rust_trainer_b200 import dp, synth

    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=1)
    flat, loss, b = _grads(_examples(spec), rank, world)
    g = torch.from_numpy(flat)
    dp.allreduce_sum_(g)
    lt = torch.tensor([loss], dtype=torch.float64)
    dp.allreduce_sum_(lt)
    out[rank] = (g.numpy().copy(), float(lt[0]), b.indices, b.batch_tokens)
    dist.destroy_process_group()


def test_two_ranks_equal_one():
    from oracle import oracle as O
    from rust_trainer_b200 import synth

    O.lib()  # build once before forking workers
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        results = dict(out)
    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=1)
    full, loss, b = _grads(_examples(spec), 0, 1)
    assert b.indices == [0, 1, 2, 3, 4] and b.batch_tokens == sum(n - 5 for n in (12, 9, 12, 7, 11))
    assert results[0][2] == [0, 2, 4] and results[1][2] == [1, 3]
    for r in range(world):
        g, l, _, bt = results[r]
        assert bt == b.batch_tokens  # the weight is the GLOBAL 1/batch_tokens on every rank
        assert np.linalg.norm(g - full) / np.linalg.norm(full) < 1e-5  # the bar for N GPUs vs 1
        assert abs(l - loss) < 1e-5 * abs(loss)
    assert np.array_equal(results[0][0], results[1][0])  # every rank holds the same reduced gradient


def test_local_batch_edges():
    from rust_trainer_b200 import dp

    ex = [(np.arange(6, dtype=np.int32), 3), (np.arange(4, dtype=np.int32), 0)]
    b = dp.local_batch(ex, 1, 4)  # more ranks than sequences: rank 1 gets the second, ranks 2, 3 nothing
    assert b.indices == [1] and b.batch_tokens == 3 + 3 and list(b.target_pos) == [0, 1, 2]
    e = dp.local_batch(ex, 3, 4)
    assert e.seqs == [] and e.target_pos.size == 0 and e.batch_tokens == 6
    try:
        dp.shard_sequences(4, 4, 4)
        raise AssertionError("rank outside the world accepted")
    except ValueError:
        pass
