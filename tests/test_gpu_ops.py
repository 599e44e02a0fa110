"""One device operation at a time against the CPU oracle's restatement of the same reference
function (src/ops.rs, src/attention.rs, src/model.rs), through the op-level C ABI.

Tolerances: the device kernels emit the f16 inputs of the next matmul (11 significant bits), so
element-wise results are compared at 2e-3 of the tensor's largest magnitude and whole tensors at
rel-L2 1e-3; f32 outputs (rmsnorm backward, attention gradients) at rel-L2 2e-3 because their
inputs were rounded to f16 on the way in; log-probabilities at 1e-5 absolute.
"""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import oracle as O
from rust_trainer_b200 import ops

pytestmark = pytest.mark.gpu


def _close16(got, want, tol=2e-3, floor=0.0):
    """`floor`: absolute slack for values below what an f16 row times its factor can hold."""
    scale = float(np.abs(want).max()) + 1e-30
    assert float(np.abs(got - want).max()) <= tol * scale + floor, (float(np.abs(got - want).max()), scale)
    assert np.linalg.norm(got.astype(np.float64) - want) <= 1e-3 * np.linalg.norm(want.astype(np.float64)) + floor * np.sqrt(got.size)


@pytest.mark.parametrize("rows,d", [(1, 128), (37, 896), (64, 1024), (5, 2560), (33, 3072), (3, 100)])
def test_rmsnorm_forward_and_backward(ctx, rows, d):
    rng = np.random.default_rng(rows * 7 + d)
    x = (rng.standard_normal((rows, d)) * rng.uniform(0.1, 30.0, (rows, 1))).astype(np.float32)
    w = (1.0 + rng.uniform(-0.3, 0.3, d)).astype(np.float32)
    dy = rng.standard_normal((rows, d)).astype(np.float32)
    y_o, inv = O.rmsnorm(x, w, 1e-6)
    _close16(ops.rmsnorm(ctx, x, w, 1e-6), y_o)
    dx_o = O.rmsnorm_backward(x, w, inv, dy)
    assert rel_l2(ops.rmsnorm_backward(ctx, x, w, dy, 1e-6), dx_o) < 1e-5


ROPE_CASES = [
    # nh, nkv, hd, rot, neox, theta, factors, qk_norm
    (16, 8, 128, 128, True, 1e6, False, True),     # Qwen3-0.6B heads
    (14, 2, 64, 64, True, 1e6, False, False),      # Qwen2.5-0.5B heads
    (24, 8, 128, 128, False, 5e5, True, False),    # Llama-3.2-3B heads, interleaved pairs, rope_freqs divisors
    (32, 8, 128, 128, True, 1e6, False, True),     # Qwen3-4B heads
    (4, 2, 64, 32, True, 1e4, False, True),        # partial rotation
]


@pytest.mark.parametrize("nh,nkv,hd,rot,neox,theta,use_factors,qk_norm", ROPE_CASES)
def test_qk_norm_rope_forward_and_backward(ctx, nh, nkv, hd, rot, neox, theta, use_factors, qk_norm):
    from rust_trainer_b200 import synth

    rng = np.random.default_rng(nh * 100 + hd)
    M = 70
    pos = np.concatenate([np.arange(40), np.arange(30)]).astype(np.int32)  # two sequences
    pos[-1] = 2047                                                        # a far position
    q_raw = rng.standard_normal((M, nh, hd)).astype(np.float32) * 3
    k_raw = rng.standard_normal((M, nkv, hd)).astype(np.float32) * 3
    v_raw = rng.standard_normal((M, nkv, hd)).astype(np.float32)
    factors = synth.llama3_rope_factors(rot, theta, 32.0) if use_factors else None
    qw = (1 + rng.uniform(-0.2, 0.2, hd)).astype(np.float32) if qk_norm else None
    kw = (1 + rng.uniform(-0.2, 0.2, hd)).astype(np.float32) if qk_norm else None

    def oracle_fwd(x, w):
        if w is None:
            return x.copy(), None
        y, inv = O.rmsnorm(x.reshape(-1, hd), w, 1e-6, fused_scale=True)  # attention.rs:170-177
        return y.reshape(x.shape), inv

    qn, q_inv = oracle_fwd(q_raw, qw)
    kn, k_inv = oracle_fwd(k_raw, kw)
    q_o = O.rope_apply(qn, pos, rot, neox, theta, 1.0, factors)
    k_o = O.rope_apply(kn, pos, rot, neox, theta, 1.0, factors)
    q_g, k_g, v_g = ops.qk_norm_rope(ctx, q_raw, k_raw, v_raw, pos, rot, neox, theta, 1.0, factors, qw, kw, 1e-6)
    _close16(q_g, q_o)
    _close16(k_g, k_o)
    assert np.array_equal(v_g, v_raw.astype(np.float16).astype(np.float32))  # the f16 K/V view, attention.rs:180-185

    dq = rng.standard_normal(q_raw.shape).astype(np.float32)
    dk = rng.standard_normal(k_raw.shape).astype(np.float32)
    dv = rng.standard_normal(v_raw.shape).astype(np.float32)
    dq_o = O.rope_apply(dq, pos, rot, neox, theta, 1.0, factors, inverse=True)
    dk_o = O.rope_apply(dk, pos, rot, neox, theta, 1.0, factors, inverse=True)
    if qk_norm:
        dq_o = O.rmsnorm_backward(q_raw.reshape(-1, hd), qw, q_inv, dq_o.reshape(-1, hd)).reshape(dq.shape)
        dk_o = O.rmsnorm_backward(k_raw.reshape(-1, hd), kw, k_inv, dk_o.reshape(-1, hd)).reshape(dk.shape)
    dq_g, dk_g, dv_g = ops.qk_norm_rope_backward(ctx, dq, dk, dv, q_raw, k_raw, pos, rot, neox, theta, 1.0, factors, qw, kw, 1e-6)
    _close16(dq_g, dq_o)
    _close16(dk_g, dk_o)
    _close16(dv_g, dv)


ATTN_CASES = [
    # nh, nkv, hd, sequence lengths
    (4, 2, 128, [512]),              # four key tiles of 128
    (2, 1, 128, [2048]),             # the longest sequence of the configurations
    (14, 2, 64, [300, 77, 1]),       # Qwen2.5 heads, ragged sequences, a one-token sequence
    (4, 4, 64, [129, 128, 127]),     # boundaries one off the tile size
    (8, 2, 128, [64, 640]),          # a short and a long sequence sharing tiles
]


def _seq_start(lens):
    return np.concatenate([np.full(n, s, np.int32) for n, s in zip(lens, np.cumsum([0] + lens[:-1]))])


@pytest.mark.parametrize("nh,nkv,hd,lens", ATTN_CASES, ids=[f"{a}x{b}x{c}-{'+'.join(map(str, d))}" for a, b, c, d in ATTN_CASES])
def test_attention_forward_and_backward(ctx, nh, nkv, hd, lens):
    rng = np.random.default_rng(nh + hd + sum(lens))
    M = sum(lens)
    ss = _seq_start(lens)
    f16 = lambda a: a.astype(np.float16).astype(np.float32)  # the kernels take f16 q, k, v: give both sides the same values
    q = f16(rng.standard_normal((M, nh, hd)) * 1.5)
    k = f16(rng.standard_normal((M, nkv, hd)) * 1.5)
    v = f16(rng.standard_normal((M, nkv, hd)))
    o_o, probs = O.attn_core_forward(q, k, v, ss)
    o_g, lse = ops.attention(ctx, q, k, v, ss)
    _close16(o_g, o_o)
    # the log-sum-exp the backward recomputes P from: check it against the oracle's scores
    i = M - 1
    s_row = (q[i, 0] / np.sqrt(hd)) @ k[ss[i]:i + 1, 0].T
    assert abs(lse[0, i] - (s_row.max() + np.log(np.exp(s_row - s_row.max()).sum()))) < 2e-3
    d_o = (rng.standard_normal((M, nh, hd)) * rng.uniform(1e-4, 10.0, (M, 1, 1))).astype(np.float32)  # row scales over 5 decades
    dq_o, dk_o, dv_o = O.attn_core_backward(q, k, v, probs, d_o, ss)
    dq_g, dk_g, dv_g = ops.attention_backward(ctx, q, k, v, d_o, ss)
    assert rel_l2(dq_g, dq_o) < 2e-3 and rel_l2(dk_g, dk_o) < 2e-3 and rel_l2(dv_g, dv_o) < 2e-3
    # reruns give the same bits (no float atomics)
    again = ops.attention_backward(ctx, q, k, v, d_o, ss)
    assert all(np.array_equal(a, b) for a, b in zip((dq_g, dk_g, dv_g), again))


@pytest.mark.parametrize("rows,ff", [(3, 3072), (17, 4864), (9, 8192), (5, 9728), (2, 100)])
def test_swiglu_forward_and_backward(ctx, rows, ff):
    rng = np.random.default_rng(rows + ff)
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    g = f16(rng.standard_normal((rows, ff)) * 4)
    u = f16(rng.standard_normal((rows, ff)) * 2)
    dh = (rng.standard_normal((rows, ff)) * rng.uniform(1e-3, 5.0, (rows, 1))).astype(np.float32)
    _close16(ops.swiglu(ctx, g, u), O.swiglu(g, u))
    dg_o, du_o = O.swiglu_backward(g, u, dh)
    dg_g, du_g = ops.swiglu_backward(ctx, g, u, dh)
    for r in range(rows):  # the gradients carry one scale per row
        _close16(dg_g[r], dg_o[r])
        _close16(du_g[r], du_o[r])


@pytest.mark.parametrize("vocab", [151936, 128256, 1001])
def test_cross_entropy_rows_at_full_vocabulary(ctx, vocab):
    rng = np.random.default_rng(vocab)
    rows = 6
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[1, 77] = 40.0           # a confident row
    logits[2] *= 0.01              # a flat row
    logits[3, [5, vocab - 1]] = 25.0  # a tie for the maximum: argmax is the LAST index (max_by, src/eval.rs:167)
    target = np.array([3, 77, vocab - 1, 5, 0, vocab // 2], np.int32)
    weight = rng.uniform(0.1, 1.0, rows).astype(np.float32)
    res = ops.cross_entropy(ctx, logits, target, weight, want_argmax=True, want_dlogits=True)
    hits = 0
    for r in range(rows):
        lse, p = O.softmax_row(logits[r])
        assert abs(res["logp"][r] - (logits[r, target[r]] - lse)) < 1e-5 * max(1.0, abs(lse))
        hits += int(not np.any(logits[r] > logits[r, target[r]]))  # model.rs:584
        d = p.copy()
        d[target[r]] -= 1.0
        d *= weight[r]
        # p - onehot leaves the kernel as f16 (smallest step 6e-8) times the row's weight: a row the
        # model is sure of has a gradient below that step, which comes out as exact zeros
        _close16(res["dlogits"][r], d, floor=6e-8 * float(weight[r]))
        assert res["argmax"][r] == vocab - 1 - int(np.argmax(logits[r][::-1]))
    assert res["hits"] == hits


@pytest.mark.parametrize("ff", [3072, 100])
def test_swiglu_product_beyond_f16_is_an_error_not_a_nan(ctx, ff):
    """silu(gate) * up is stored in 16 bits as the input of down_proj (the reference keeps f32,
    src/model.rs Mlp::forward); a product beyond 65504 must come back as a status the host can act
    on, and the context must keep working afterwards."""
    from rust_trainer_b200._lib import RtError

    g = np.full((4, ff), 1.0, np.float32)
    u = np.full((4, ff), 2.0, np.float32)
    g[2, ff // 2], u[2, ff // 2] = 300.0, 300.0  # silu(300) * 300 = 90 000
    with pytest.raises(RtError) as e:
        ops.swiglu(ctx, g, u)
    assert e.value.status == 9
    g[2, ff // 2] = 1.0
    _close16(ops.swiglu(ctx, g, u), O.swiglu(g, u))


@pytest.mark.parametrize("lens,nh,nkv,hd,exact", [([256, 384], 4, 2, 128, True), ([128, 512, 128], 4, 4, 64, True),
                                                   ([200, 330], 4, 2, 128, False), ([64, 1, 447], 4, 4, 64, False)])
def test_attention_backward_of_a_sequence_ignores_its_batch_mates(ctx, lens, nh, nkv, hd, exact):
    """What a sequence's backward computes may not depend on the other sequences of the batch: rows
    are weighed against the largest gradient factor of their OWN sequence.  The sequences differ in
    gradient magnitude by decades.  To the last bit when every sequence starts on a tile boundary
    (128 tokens: the kernels tile the batch, not the sequence); otherwise a sequence's tiles fall
    differently and the f32 sums differ in their last digits."""
    rng = np.random.default_rng(sum(lens))
    M = sum(lens)
    ss = _seq_start(lens)
    q = rng.standard_normal((M, nh, hd)).astype(np.float32)
    k = rng.standard_normal((M, nkv, hd)).astype(np.float32)
    v = rng.standard_normal((M, nkv, hd)).astype(np.float32)
    d_o = rng.standard_normal((M, nh, hd)).astype(np.float32) * rng.uniform(0.1, 1.0, (M, 1, 1)).astype(np.float32)
    starts = np.cumsum([0] + lens)
    for i in range(len(lens)):
        d_o[starts[i]:starts[i + 1]] *= np.float32(10.0 ** (-1.5 * i))
    whole = ops.attention_backward(ctx, q, k, v, d_o, ss)
    for i, n in enumerate(lens):
        a, b = starts[i], starts[i + 1]
        alone = ops.attention_backward(ctx, q[a:b], k[a:b], v[a:b], d_o[a:b], np.zeros(n, np.int32))
        for w, s in zip(whole, alone):
            if exact:
                assert np.array_equal(w[a:b], s), (i, float(np.abs(w[a:b] - s).max()))
            else:
                assert rel_l2(w[a:b], s) < 1e-5, (i, rel_l2(w[a:b], s))
