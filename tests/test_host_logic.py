"""Host-side logic: synthetic model shapes, targets, data-parallel sharding."""
import numpy as np
import pytest

from rust_trainer_b200 import dp, quants as Q, synth


def test_preset_sizes_match_the_configs():
    s = synth.preset("qwen3-0.6b")
    assert s.frozen_params_per_layer() * s.n_layers == 440_401_920
    assert sum(16 * (r + c) for r, c in s.linear_shapes().values()) * s.n_layers == 10_092_544
    s = synth.preset("qwen2.5-0.5b")
    assert s.frozen_params_per_layer() * s.n_layers == 357_826_560
    s = synth.preset("llama-3.2-3b")
    assert s.frozen_params_per_layer() * s.n_layers == 2_818_572_288
    s = synth.preset("qwen3-4b")
    assert s.frozen_params_per_layer() * s.n_layers == 3_633_315_840


def test_k_quant_fallback_per_tensor():
    s = synth.preset("qwen2.5-0.5b", quant="Q4_K", fallback_quant="Q4_0")
    assert s.quant_for(896) == Q.Q4_0 and s.quant_for(4864) == Q.Q4_K


def test_answer_targets_rule():
    toks = np.arange(10, dtype=np.int32)
    tp, tt = synth.answer_targets(toks, 6)
    assert list(tp) == [5, 6, 7, 8] and list(tt) == [6, 7, 8, 9]
    tp, tt = synth.answer_targets(toks, 0)  # answer_start.max(1)
    assert tp[0] == 0 and tt[0] == 1 and tp.size == 9


def test_tensor_names_and_shapes():
    spec = synth.preset("tiny-qwen2", quant="Q8_0")
    T = synth.build_tensors(spec)
    assert "blk.0.attn_q.bias" in T and "blk.1.ffn_down.weight" in T and "output.weight" not in T
    t, rows, cols, arr = T["blk.0.ffn_down.weight"]
    assert (rows, cols) == (spec.hidden, spec.ff) and arr.shape == (rows, Q.row_bytes(t, cols))
    spec = synth.preset("tiny-llama")
    T = synth.build_tensors(spec)
    assert "output.weight" in T and T["rope_freqs.weight"][3].size == spec.rot_dim // 2


def test_llama3_rope_factor_rule():
    f = synth.llama3_rope_factors(128, 5e5, 32.0)
    assert f[0] == 1.0 and f[-1] == 32.0 and np.all(np.diff(f) >= 0)


def test_lora_order_is_block_major():
    spec = synth.preset("tiny-qwen3")
    ads = synth.lora_adapters(spec, 4, 8.0, 1)
    assert [a["name"] for a in ads[:8]] == [f"blk.0.{n}" for n in synth.LINEARS] + ["blk.1.attn_q"]


def test_shard_sequences_round_robin():
    assert dp.shard_sequences(10, 0, 4) == [0, 4, 8]
    assert dp.shard_sequences(10, 3, 4) == [3, 7]
    assert sorted(sum((dp.shard_sequences(7, r, 3) for r in range(3)), [])) == list(range(7))
    with pytest.raises(ValueError):
        dp.shard_sequences(4, 4, 4)


def test_objective_helpers():
    """softplus with torch's threshold (src/tensor.rs:146-153), sigmoid, and the batch layout of
    answer targets (global positions, per-example spans)."""
    from rust_trainer_b200 import objectives as obj

    assert abs(obj.softplus(0.0) - np.log(2.0)) < 1e-6 and obj.softplus(25.0) == 25.0 and obj.softplus(-30.0) < 1e-12
    assert obj.sigmoid(0.0) == 0.5 and abs(obj.sigmoid(2.0) + obj.sigmoid(-2.0) - 1.0) < 1e-6
    seqs, tp, tt, spans = obj._layout([(np.arange(10), 6), (np.arange(8), 0)])
    assert [s.size for s in seqs] == [10, 8] and spans == [(0, 4), (4, 11)]
    assert tp.tolist() == [5, 6, 7, 8] + [10 + i for i in range(7)]  # i >= max(answer_start, 1) predicts from i - 1
    assert tt.tolist() == [6, 7, 8, 9] + list(range(1, 8))


def test_pack_shared_prompt():
    """pack (src/model.rs:266-290): longest common prefix, at least one own token per sequence,
    a single sequence shares nothing; Packed::index / map_targets."""
    from rust_trainer_b200 import packing

    a, b, c = np.array([1, 2, 3, 4, 5]), np.array([1, 2, 3, 9]), np.array([1, 2, 3, 7, 8, 6])
    p = packing.pack([a, b, c])
    assert p.shared == 3 and p.offsets == [3, 5, 6]
    assert p.tokens.tolist() == [1, 2, 3, 4, 5, 9, 7, 8, 6]
    assert p.positions.tolist() == [0, 1, 2, 3, 4, 3, 3, 4, 5]
    assert p.segments.tolist() == [0, 0, 0, 1, 1, 2, 3, 3, 3]
    assert p.index(1, 2) == 2 and p.index(1, 3) == 5 and p.index(2, 5) == 8
    assert packing.pack([a]).shared == 0
    assert packing.pack([a, a]).shared == 4  # every sequence keeps one token of its own
    tp, tt = p.map_targets(2, [2, 3, 4], [7, 8, 6])
    assert tp.tolist() == [2, 6, 7] and tt.tolist() == [7, 8, 6]
