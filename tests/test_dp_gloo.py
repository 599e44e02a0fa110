"""Data-parallel step on CPU ranks (gloo, world_size 2): sequences sharded round-robin, one
all-reduce of the flat gradient buffer, identical optimiser step on every rank.  The compute is
the CPU oracle; what is tested is the host-side sharding / weighting / all-reduce logic the GPU
path uses unchanged."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from rust_trainer_b200 import dp, synth

    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=1)
    m = O.OracleModel(spec.config(), synth.build_tensors(spec))
    m.attach_lora(synth.lora_adapters(spec, 4, 8.0, 2, b_std=0.02))
    toks = synth.token_batch(spec, 5, 12, 4)
    a0 = 6
    bt = dp.global_batch_tokens([12 - a0] * 5)
    m.zero_grad()
    loss = 0.0
    for s in dp.shard_sequences(5, rank, world):
        tp, tt = synth.answer_targets(toks[s], a0)
        lp, _ = m.forward_backward(toks[s], tp, tt, np.full(tp.size, 1.0 / bt, np.float32))
        loss += -float(lp.sum()) / bt
    flat = torch.from_numpy(np.concatenate([np.concatenate([e["ga"].ravel(), e["gb"].ravel()]) for e in m.lora]))
    dp.allreduce_sum_(flat)
    lt = torch.tensor([loss], dtype=torch.float64)
    dp.allreduce_sum_(lt)
    out[rank] = (flat.numpy().copy(), float(lt[0]))
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
    m = O.OracleModel(spec.config(), synth.build_tensors(spec))
    m.attach_lora(synth.lora_adapters(spec, 4, 8.0, 2, b_std=0.02))
    toks = synth.token_batch(spec, 5, 12, 4)
    m.zero_grad()
    loss = 0.0
    for s in range(5):
        tp, tt = synth.answer_targets(toks[s], 6)
        lp, _ = m.forward_backward(toks[s], tp, tt, np.full(tp.size, 1.0 / 30, np.float32))
        loss += -float(lp.sum()) / 30
    full = np.concatenate([np.concatenate([e["ga"].ravel(), e["gb"].ravel()]) for e in m.lora])
    for r in range(world):
        g, l = results[r]
        assert np.linalg.norm(g - full) / np.linalg.norm(full) < 1e-5
        assert abs(l - loss) < 1e-5 * abs(loss)
    assert np.array_equal(results[0][0], results[1][0])  # every rank holds the same reduced gradient
