"""adapter.gguf round trip and bit-exact resume (reference tests/engine.rs:205-255: train, write
adapter.gguf, reload, equal log-probabilities; tests/training.rs:80-113: pause/resume identical)."""
import numpy as np
import pytest

import rust_trainer_b200 as rt
from rust_trainer_b200 import adapter, synth

pytestmark = pytest.mark.gpu


def _model(ctx, spec, tensors, seed):
    m = rt.Model(ctx, spec.config(), tensors)
    m.attach_lora(8, 16.0, None, seed)
    return m


def _batch(spec):
    toks = synth.token_batch(spec, 2, 40, 7)
    tp = np.concatenate([synth.answer_targets(toks[s], 20)[0] + 40 * s for s in range(2)])
    tt = np.concatenate([synth.answer_targets(toks[s], 20)[1] for s in range(2)])
    return [toks[0], toks[1]], tp, tt, np.full(tp.size, 1.0 / tp.size, np.float32)


def _train(m, batch, steps, lr=5e-3):
    seqs, tp, tt, w = batch
    for _ in range(steps):
        m.zero_grad()
        m.forward_backward(seqs, tp, tt, w)
        m.optim_step(lr, 1.0, weight_decay=0.01)


def test_adapter_gguf_round_trip(ctx, tmp_path):
    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=4, w_std=0.05)
    tensors = synth.build_tensors(spec)
    batch = _batch(spec)
    m = _model(ctx, spec, tensors, seed=1)
    _train(m, batch, 3)  # B leaves zero, so the adapter changes the outputs
    lp_trained, _, _ = m.score(batch[0], batch[1], batch[2])
    path = tmp_path / adapter.GGUF_ADAPTER_FILE
    adapter.write_gguf_adapter(m, str(path), spec.arch)

    import gguf

    r = gguf.GGUFReader(str(path))
    names = {t.name: [int(d) for d in t.shape] for t in r.tensors}
    assert names["blk.0.attn_q.weight.lora_a"] == [spec.hidden, 8]                      # ne [in, r]
    assert names["blk.0.attn_q.weight.lora_b"] == [8, spec.n_heads * spec.head_dim]     # ne [r, out]
    assert len(names) == 2 * 7 * spec.n_layers

    fresh = _model(ctx, spec, tensors, seed=2)  # different init
    lp_fresh, _, _ = fresh.score(batch[0], batch[1], batch[2])
    assert not np.array_equal(lp_fresh, lp_trained)
    assert adapter.read_gguf_adapter(fresh, str(path), spec.arch) == 7 * spec.n_layers
    lp_loaded, _, _ = fresh.score(batch[0], batch[1], batch[2])
    assert np.array_equal(lp_loaded, lp_trained)  # exact, as the reference's round trip is
    with pytest.raises(ValueError):
        adapter.read_gguf_adapter(fresh, str(path), "llama")
    m.close()
    fresh.close()


def test_resume_from_checkpoint_is_bit_identical(ctx, tmp_path):
    spec = synth.preset("tiny-qwen2", quant="Q8_0", seed=5, w_std=0.05)
    tensors = synth.build_tensors(spec)
    batch = _batch(spec)
    a = _model(ctx, spec, tensors, seed=3)
    _train(a, batch, 2)
    ck = tmp_path / "ckpt.npz"
    adapter.save_checkpoint(a, str(ck), {"step": 2, "losses": [1.0, 0.9]})
    _train(a, batch, 2)
    b = _model(ctx, spec, tensors, seed=99)
    state = adapter.load_checkpoint(b, str(ck))
    assert state["step"] == 2 and state["opt_t"] == 2
    _train(b, batch, 2)
    for la, lb in zip(a.lora_linears(), b.lora_linears()):
        pa, pb = la.lora(), lb.lora()
        assert np.array_equal(pa["a"], pb["a"]) and np.array_equal(pa["b"], pb["b"])
    ta, ma, va = a.optim_state()
    tb, mb, vb = b.optim_state()
    assert ta == tb == 4 and np.array_equal(ma, mb) and np.array_equal(va, vb)
    a.close()
    b.close()
