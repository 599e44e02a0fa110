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


def test_adapter_file_decides_alpha_and_modules(ctx, tmp_path):
    """read_gguf_adapter (src/rie.rs:369-411) rebuilds the adapters from the file: its alpha (the
    rank when the key is 0), its rank, and only the modules it names; everything else ends up
    without an adapter."""
    import gguf

    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=4, w_std=0.05)
    tensors = synth.build_tensors(spec)
    batch = _batch(spec)
    src = rt.Model(ctx, spec.config(), tensors)
    src.attach_lora(4, 32.0, ["q_proj", "ffn_down"], 5)  # alpha 32 on rank 4: scale 8
    for lin in src.lora_linears():                       # non-zero B, so the scale matters
        lo = lin.lora()
        lin.write_lora(lo["a"], np.random.default_rng(1).standard_normal(lo["b"].shape).astype(np.float32) * 0.05)
    want = src.score(batch[0], batch[1], batch[2])[0]
    path = tmp_path / adapter.GGUF_ADAPTER_FILE
    adapter.write_gguf_adapter(src, str(path), spec.arch)
    dst = _model(ctx, spec, tensors, seed=9)  # rank 8, alpha 16, all seven projections
    assert adapter.read_gguf_adapter(dst, str(path), spec.arch) == 2 * spec.n_layers
    assert [l.name for l in dst.lora_linears()] == [l.name for l in src.lora_linears()]
    assert all(l.rank == 4 for l in dst.lora_linears())
    assert np.array_equal(dst.score(batch[0], batch[1], batch[2])[0], want)
    # alpha 0 in the file means alpha = rank (scale 1)
    w = gguf.GGUFWriter(str(tmp_path / "zero.gguf"), spec.arch)
    w.add_string("general.type", "adapter")
    w.add_string("adapter.type", "lora")
    w.add_float32("adapter.lora.alpha", 0.0)
    for lin in src.lora_linears():
        lo = lin.lora()
        w.add_tensor(f"{lin.name}.weight.lora_a", lo["a"])
        w.add_tensor(f"{lin.name}.weight.lora_b", lo["b"])
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    adapter.read_gguf_adapter(dst, str(tmp_path / "zero.gguf"), spec.arch)
    src.attach_lora(4, 4.0, ["q_proj", "ffn_down"], 5)
    for a, b in zip(src.lora_linears(), dst.lora_linears()):
        lo = b.lora()
        a.write_lora(lo["a"], lo["b"])
    assert np.array_equal(dst.score(batch[0], batch[1], batch[2])[0], src.score(batch[0], batch[1], batch[2])[0])
    src.close()
    dst.close()


def test_resume_from_checkpoint_is_bit_identical(ctx, tmp_path):
    spec = synth.preset("tiny-qwen2", quant="Q8_0", seed=5, w_std=0.05)
    tensors = synth.build_tensors(spec)
    batch = _batch(spec)
    a = _model(ctx, spec, tensors, seed=3)
    _train(a, batch, 2)
    ck = tmp_path / "checkpoint.safetensors"
    fp = adapter.data_fingerprint([(s, 20) for s in batch[0]])
    run = {"data_fingerprint": fp, "config_json": '{"rank":8,"alpha":16.0}'}
    adapter.save_checkpoint(a, str(ck), dict(run, step=2, losses=[1.0, 0.9]))
    # the file is the trainer's own layout (src/train.rs:389-406): <name>.A|B, .adam_m, .adam_v, metadata trainer_state
    from safetensors import safe_open

    with safe_open(str(ck), framework="numpy") as f:
        keys = set(f.keys())
        assert {"blk.0.attn_q.A", "blk.0.attn_q.A.adam_m", "blk.0.attn_q.B.adam_v", "blk.1.ffn_down.B"} <= keys
        assert len(keys) == 3 * 2 * 7 * spec.n_layers and "trainer_state" in f.metadata()
        assert f.get_tensor("blk.0.attn_q.A").shape == (8 * spec.hidden,)
    _train(a, batch, 2)
    b = _model(ctx, spec, tensors, seed=99)
    with pytest.raises(ValueError, match="training data changed"):  # src/train.rs:414-416
        adapter.load_checkpoint(b, str(ck), dict(run, data_fingerprint=fp ^ 1))
    with pytest.raises(ValueError, match="training config changed"):  # src/train.rs:417-419
        adapter.load_checkpoint(b, str(ck), dict(run, config_json="{}"))
    state = adapter.load_checkpoint(b, str(ck), run)
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
