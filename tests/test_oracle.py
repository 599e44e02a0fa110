"""The CPU oracle against the reference's own known answers and invariants
(reference tests cited per case)."""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import oracle as O
from rust_trainer_b200 import quants as Q
from rust_trainer_b200 import synth
from rust_trainer_b200.model import schedule_lr
from rust_trainer_b200.rng import Rng


def test_schedule_known_answers():
    # src/optim.rs:118-123
    for f in (O.schedule_lr, schedule_lr):
        assert abs(f(1.0, 10, 110, 0.1, 0) - 0.1) < 1e-6
        assert abs(f(1.0, 10, 110, 0.1, 9) - 1.0) < 1e-6
        assert abs(f(1.0, 10, 110, 0.1, 10) - 1.0) < 1e-6
        assert abs(f(1.0, 10, 110, 0.1, 110) - 0.1) < 1e-6
        assert 0.5 < f(1.0, 10, 110, 0.1, 60) < 0.6
    for step in range(0, 130, 7):
        assert abs(O.schedule_lr(3e-4, 2, 20, 0.1, step) - schedule_lr(3e-4, 2, 20, 0.1, step)) < 1e-9


def test_round_f16_matches_ieee_conversion():
    # tests/engine.rs:265-276: 20k values and the listed edge inputs
    edge = [0.0, -0.0, 65504.0, 1e-8, 6.1e-5, 2049.0, 2051.0]
    rng = np.random.default_rng(1)
    vals = np.concatenate([np.array(edge, np.float32), (rng.standard_normal(20000) * 10 ** rng.uniform(-6, 4, 20000)).astype(np.float32)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).astype(np.float32)
    got = np.array([O.round_f16(float(v)) for v in vals], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_rng_restatement_matches_oracle_stream():
    a, b = O.Rng(1234), Rng(1234)
    assert a.next_u64() == b.next_u64()
    assert np.array_equal(a.vec_uniform_sym(1000, 0.03125), b.uniform_sym(1000, 0.03125))
    assert np.abs(a.vec_normal(999, 0.5) - b.normal(999, 0.5)).max() < 1e-6
    assert a.next_u64() == b.next_u64()  # both consumed the same number of draws
    v1, v2 = list(range(20)), list(range(20))
    r1, r2 = Rng(7), O.Rng(7)
    r1.shuffle(v1)
    for i in range(19, 0, -1):
        j = r2.next_u64() % (i + 1)
        v2[i], v2[j] = v2[j], v2[i]
    assert v1 == v2


@pytest.mark.parametrize("t", [Q.F16, Q.Q8_0, Q.Q4_0, Q.Q4_K, Q.Q6_K])
def test_adjoint_identity(t):
    # src/frozen.rs:218-227: <dy, x.W^T> == <dy.W, x>
    rng = np.random.default_rng(3)
    n, k, m = 96, 256, 5
    packed = Q.quantize((rng.standard_normal((n, k)) * 0.1).astype(np.float32), t)
    x = rng.standard_normal((m, k)).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    y = O.frozen_forward(t, n, k, packed, x, m)
    dx = np.zeros((m, k), np.float32)
    O.frozen_backward_input(t, n, k, packed, dy, m, dx)
    lhs, rhs = float((dy.astype(np.float64) * y).sum()), float((dx.astype(np.float64) * x).sum())
    assert abs(lhs - rhs) <= 1e-3 * max(1.0, abs(lhs))
    # backward_input equals the dense product built from row() (tests/engine.rs:96-120)
    w = O.dequant_rows(t, packed, n, k)
    assert rel_l2(dx, dy @ w) < 1e-5
    # and it accumulates
    O.frozen_backward_input(t, n, k, packed, dy, m, dx)
    assert rel_l2(dx, 2 * (dy @ w)) < 1e-5


def test_softmax_row_f64_normaliser():
    rng = np.random.default_rng(0)
    logits = (rng.standard_normal(151936) * 2).astype(np.float32)
    lse, p = O.softmax_row(logits)
    ref = np.log(np.exp(logits.astype(np.float64) - logits.max()).sum()) + logits.max()
    assert abs(lse - ref) < 2e-6 * abs(ref)
    assert abs(p.astype(np.float64).sum() - 1.0) < 1e-5


@pytest.mark.parametrize("name", ["tiny-qwen3", "tiny-qwen2", "tiny-llama"])
def test_lora_gradients_match_finite_differences(name):
    # tests/gradcheck.rs:179-253: central differences, eps 2e-3, rtol 3e-2, atol 3e-4
    spec = synth.preset(name, quant="Q8_0", w_std=0.15, seed=3)
    tensors = synth.build_tensors(spec)
    synth.perturb_norms(tensors, 5)
    cfg = spec.config()
    cfg["kv_f16"] = False  # the f16 rounding of K/V is a step function; gradcheck.rs runs without it
    m = O.OracleModel(cfg, tensors)
    m.attach_lora(synth.lora_adapters(spec, 4, 8.0, seed=7, b_std=0.05))
    toks = synth.token_batch(spec, 1, 12, 1)[0]
    tp, tt = synth.answer_targets(toks, 5)
    w = np.full(tp.size, 1.0 / tp.size, np.float32)
    m.zero_grad()
    m.forward_backward(toks, tp, tt, w)

    def loss():
        lp, _, _ = m.score(toks, tp, tt)
        return float(-(lp.astype(np.float64) * w).sum())

    rng = np.random.default_rng(0)
    eps = 2e-3
    for ei in (0, 3, 6, 7, 13):
        e = m.lora[ei]
        for key, gk in (("a", "ga"), ("b", "gb")):
            for _ in range(2):
                idx = tuple(rng.integers(0, s) for s in e[key].shape)
                old = e[key][idx]
                e[key][idx] = old + eps
                lp = loss()
                e[key][idx] = old - eps
                lm = loss()
                e[key][idx] = old
                fd = (lp - lm) / (2 * eps)
                assert abs(fd - e[gk][idx]) <= 3e-4 + 3e-2 * abs(fd), (ei, key, idx, fd, e[gk][idx])


def test_batch_of_sequences_equals_one_at_a_time():
    # the trainer accumulates per example (src/train.rs:339-351); a concatenated batch with
    # per-sequence causal masks must give the same numbers (cf. tests/gradcheck.rs:279-338)
    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=1)
    tensors = synth.build_tensors(spec)
    m = O.OracleModel(spec.config(), tensors)
    m.attach_lora(synth.lora_adapters(spec, 4, 8.0, 2))
    toks = synth.token_batch(spec, 3, 10, 4)
    m.zero_grad()
    lps = []
    for s in range(3):
        tp, tt = synth.answer_targets(toks[s], 4)
        lps.append(m.forward_backward(toks[s], tp, tt, np.full(tp.size, 0.1, np.float32))[0])
    g1 = [e["ga"].copy() for e in m.lora]
    m.zero_grad()
    seg = np.repeat(np.arange(3) * 10, 10).astype(np.int32)
    tps, tts = zip(*[(synth.answer_targets(toks[s], 4)[0] + 10 * s, synth.answer_targets(toks[s], 4)[1]) for s in range(3)])
    lp, _ = m.forward_backward(toks.reshape(-1), np.concatenate(tps), np.concatenate(tts), np.full(18, 0.1, np.float32), seg_start=seg)
    assert np.abs(lp - np.concatenate(lps)).max() < 1e-5
    assert max(rel_l2(e["ga"], a) for a, e in zip(g1, m.lora)) < 1e-5


def test_oracle_reproduces_committed_fixture():
    import os
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from make_golden import tiny_model_case

    spec, tensors, adapters, toks = tiny_model_case()
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "tiny_model.npz"))
    om = O.OracleModel(spec.config(), tensors)
    om.attach_lora(adapters)
    om.zero_grad()
    lps = []
    for s in range(2):
        tp, tt = synth.answer_targets(toks[s], 24)
        lps.append(om.forward_backward(toks[s], tp, tt, np.full(tp.size, 1.0 / 48, np.float32))[0])
    grads = np.concatenate([np.concatenate([e["ga"].ravel(), e["gb"].ravel()]) for e in om.lora])
    assert np.abs(np.concatenate(lps) - gold["logp"]).max() < 1e-5
    assert rel_l2(grads, gold["grads"]) < 1e-5


def test_loss_is_linear_in_weights():
    # tests/gradcheck.rs:257-275
    spec = synth.preset("tiny-qwen3", quant="F16", seed=2)
    m = O.OracleModel(spec.config(), synth.build_tensors(spec))
    m.attach_lora(synth.lora_adapters(spec, 4, 8.0, 3, b_std=0.05))
    toks = synth.token_batch(spec, 1, 16, 5)[0]
    tp, tt = synth.answer_targets(toks, 8)
    m.zero_grad()
    m.forward_backward(toks, tp, tt, np.full(tp.size, 0.25, np.float32))
    g1 = m.lora[0]["ga"].copy()
    m.zero_grad()
    m.forward_backward(toks, tp, tt, np.full(tp.size, 0.5, np.float32))
    assert rel_l2(m.lora[0]["ga"], 2 * g1) < 1e-5


@pytest.mark.parametrize("t", [Q.Q8_0, Q.Q4_0, Q.Q4_K, Q.Q6_K, Q.F16])
def test_int8_activation_mode_bounds_the_rounding(t):
    # src/rie.rs:77-80: the engine's forward rounds activations to 8 bits per block.  Mode (ii)
    # restates that rounding; it moves a forward product by at most the rounding's own size
    # (half a step of amax/127 per element: about 0.5 % of the row in rel-L2), leaves 16-bit
    # weights and the backward alone, and is off again afterwards.
    rng = np.random.default_rng(5)
    n, k, m = 64, 512, 7
    packed = Q.quantize((rng.standard_normal((n, k)) * 0.1).astype(np.float32), t)
    x = rng.standard_normal((m, k)).astype(np.float32)
    smooth = O.frozen_forward(t, n, k, packed, x, m)
    try:
        O.set_act_int8(True)
        rounded = O.frozen_forward(t, n, k, packed, x, m)
        dx = np.zeros((m, k), np.float32)
        O.frozen_backward_input(t, n, k, packed, smooth, m, dx)
    finally:
        O.set_act_int8(False)
    if t == Q.F16:
        assert np.array_equal(rounded, smooth)
    else:
        assert 1e-4 < rel_l2(rounded, smooth) < 2e-2
    dx0 = np.zeros((m, k), np.float32)
    O.frozen_backward_input(t, n, k, packed, smooth, m, dx0)
    assert np.array_equal(dx, dx0)
    assert np.array_equal(O.frozen_forward(t, n, k, packed, x, m), smooth)
