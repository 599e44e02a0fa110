"""Shared-prompt packed batches on the GPU (src/model.rs:234-290, forward_backward_packed): the
packed pass equals running the examples separately (the reference's own check,
tests/gradcheck.rs:327-333), here against the per-example oracle at the north-star tolerances."""
import numpy as np
import pytest

import rust_trainer_b200 as rt
from conftest import cosine, rel_l2
from rust_trainer_b200 import packing, synth
from test_gpu_model import GRAD_COS, GRAD_TOL, LOSS_TOL, _flat, _gpu_flat, _setup

pytestmark = pytest.mark.gpu


def _family(spec, rng, prompt_len, tails):
    prompt = rng.integers(0, spec.vocab, prompt_len).astype(np.int32)
    return [np.concatenate([prompt, rng.integers(0, spec.vocab, n).astype(np.int32)]) for n in tails]


@pytest.mark.parametrize("name,quant", [("tiny-qwen3", "Q8_0"), ("tiny-llama", "Q4_0")])
def test_packed_equals_separate(ctx, name, quant):
    spec, om, gm = _setup(ctx, name, quant)
    rng = np.random.default_rng(5)
    families = [_family(spec, rng, 70, [20, 33, 9]), _family(spec, rng, 3, [40]), _family(spec, rng, 30, [65, 70])]
    starts = [[60, 75, 70], [10], [30, 31]]  # answer starts: inside the prompt, at its end, after it
    groups = [packing.pack(f) for f in families]
    assert groups[0].shared == 70 and groups[1].shared == 0 and groups[2].shared == 30
    # per-example targets, and the same targets mapped into the packed batch
    per_ex, tp_packed, tt_packed, off = [], [], [], 0
    for fam, st, g in zip(families, starts, groups):
        for k, (seq, a) in enumerate(zip(fam, st)):
            tp, tt = synth.answer_targets(seq, a)
            per_ex.append((seq, tp, tt))
            mp, mt = g.map_targets(k, tp, tt)
            tp_packed.append(mp + off)
            tt_packed.append(mt)
        off += g.tokens.size
    tp_packed, tt_packed = np.concatenate(tp_packed), np.concatenate(tt_packed)
    n_t = tp_packed.size
    w = np.full(n_t, 1.0 / n_t, np.float32)
    # the examples one at a time on the oracle
    om.zero_grad()
    lp_o, k = [], 0
    for seq, tp, tt in per_ex:
        lp_o.append(om.forward_backward(seq, tp, tt, w[k:k + tp.size])[0])
        k += tp.size
    lp_o = np.concatenate(lp_o)
    go = _flat(om.lora, "ga", "gb")
    # packed on the GPU
    gm.zero_grad()
    lp_p, _ = gm.forward_backward_packed(groups, tp_packed, tt_packed, w)
    gp = _gpu_flat(gm, "ga", "gb")
    assert np.max(np.abs(lp_p - lp_o) / np.abs(lp_o)) < LOSS_TOL
    assert rel_l2(gp, go) < GRAD_TOL and cosine(gp, go) > GRAD_COS
    # and the GPU's own separate pass
    seqs = [e[0] for e in per_ex]
    offs = np.cumsum([0] + [s.size for s in seqs])
    tp_s = np.concatenate([e[1] + o for e, o in zip(per_ex, offs)])
    gm.zero_grad()
    lp_s, _ = gm.forward_backward(seqs, tp_s, tt_packed, w)
    gs = _gpu_flat(gm, "ga", "gb")
    assert np.max(np.abs(lp_p - lp_s) / np.abs(lp_s)) < LOSS_TOL and rel_l2(gp, gs) < 3e-3
    # forward only
    lp_f, _ = gm.score_packed(groups, tp_packed, tt_packed)
    assert np.max(np.abs(lp_f - lp_p)) < 1e-5
    gm.close()
    om.close()


def test_bad_layouts_are_refused(ctx):
    spec, om, gm = _setup(ctx, "tiny-qwen3", "Q4_0")
    g = packing.pack([np.arange(12, dtype=np.int32), np.concatenate([np.arange(6), np.arange(20, 26)]).astype(np.int32)])
    bad = packing.Packed(g.tokens, g.positions, g.segments.copy(), g.shared, g.offsets)
    bad.segments[-1] = 5  # runs must count up by one
    with pytest.raises(rt.RtError):
        gm.forward_backward_packed([bad], [3], [1], [1.0])
    bad2 = packing.Packed(g.tokens, g.positions.copy(), g.segments, g.shared, g.offsets)
    bad2.positions[0] = -1
    with pytest.raises(rt.RtError):
        gm.forward_backward_packed([bad2], [3], [1], [1.0])
    gm.close()
    om.close()
