"""Linear + LoRA on the GPU against the oracle's restatement of src/linear.rs:73-121.

Tolerances: outputs and dx 2e-3 relative L2 (f16 operands, f32 accumulation); adapter
gradients 5e-3 relative L2 and cosine >= 0.9999 (the north-star bar is 1e-2 / 0.999).
"""
import numpy as np
import pytest

import rust_trainer_b200 as rt
from conftest import cosine, rel_l2
from oracle import oracle as O
from rust_trainer_b200 import quants as Q

pytestmark = pytest.mark.gpu

CASES = [(Q.Q4_0, 256, 128, 50, 8), (Q.Q8_0, 3072, 1024, 700, 16), (Q.Q6_K, 512, 1024, 300, 32),
         (Q.F16, 384, 256, 100, 16), (Q.BF16, 256, 256, 65, 4), (Q.Q4_K, 1024, 768, 257, 16), (Q.Q8_0, 128, 896, 1, 64),
         # enough 256-row tiles for the CTA-pair kernel, ragged token counts, packed and 16-bit weights
         (Q.Q8_0, 1024, 512, 2500, 16), (Q.Q4_0, 512, 512, 5001, 8), (Q.F16, 768, 512, 3300, 16),
         (Q.Q6_K, 512, 1024, 4999, 32), (Q.Q4_K, 1280, 256, 2047, 64)]


def _make(ctx, rng, t, n, k, r, bias=True):
    packed = Q.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), t)
    b = (rng.standard_normal(n) * 0.01).astype(np.float32) if bias else None
    a_ = (rng.standard_normal((r, k)) / r).astype(np.float32)
    b_ = (rng.standard_normal((n, r)) * 0.05).astype(np.float32)
    f = rt.Frozen(ctx, t, n, k, packed)
    lin = rt.Linear("blk.0.test", f, b)
    lin.attach_lora(r, 2.0 * r, a_, b_)
    return packed, b, a_, b_, f, lin


@pytest.mark.parametrize("t,n,k,m,r", CASES, ids=[f"{Q.NAMES[c[0]]}-{c[1]}x{c[2]}-t{c[3]}-r{c[4]}" for c in CASES])
def test_forward_backward_with_adapter(ctx, t, n, k, m, r):
    rng = np.random.default_rng(n + k + m + r)
    packed, bias, a, b, f, lin = _make(ctx, rng, t, n, k, r)
    alpha = 2.0 * r
    x = rng.standard_normal((m, k)).astype(np.float32)
    assert rel_l2(lin.forward(x, m), O.linear_forward(t, n, k, packed, bias, r, alpha, a, b, x, m)) < 2e-3
    # gradients spanning five orders of magnitude between rows: the per-row scaling must hold
    dy = (rng.standard_normal((m, n)) * 1e-3 * np.exp(rng.standard_normal((m, 1)) * 2.5)).astype(np.float32)
    dx = lin.backward(x, dy, m)
    ga, gb = np.zeros_like(a), np.zeros_like(b)
    dxo = O.linear_backward(t, n, k, packed, r, alpha, a, b, ga, gb, x, dy, m)
    got = lin.lora()
    assert rel_l2(dx, dxo) < 2e-3
    assert rel_l2(got["ga"], ga) < 5e-3 and cosine(got["ga"], ga) > 0.9999
    assert rel_l2(got["gb"], gb) < 5e-3 and cosine(got["gb"], gb) > 0.9999
    # a second backward accumulates into ga / gb (src/linear.rs:108,113)
    lin.backward(x, dy, m)
    got2 = lin.lora()
    assert rel_l2(got2["ga"], 2 * ga) < 5e-3 and rel_l2(got2["gb"], 2 * gb) < 5e-3
    lin.zero_grad()
    z = lin.lora()
    assert not z["ga"].any() and not z["gb"].any()
    lin.close()
    f.close()


def test_adapter_bypass_and_fresh_adapter_is_a_no_op(ctx):
    rng = np.random.default_rng(5)
    t, n, k, m, r = Q.Q8_0, 256, 256, 40, 8
    packed, bias, a, b, f, lin = _make(ctx, rng, t, n, k, r)
    x = rng.standard_normal((m, k)).astype(np.float32)
    base = O.linear_forward(t, n, k, packed, bias, 0, 1.0, None, None, x, m)
    lin.set_lora_enabled(False)  # src/linear.rs:64-70
    assert rel_l2(lin.forward(x, m), base) < 2e-3
    dy = rng.standard_normal((m, n)).astype(np.float32)
    lin.backward(x, dy, m)
    g = lin.lora()
    assert not g["ga"].any() and not g["gb"].any()  # no gradient while bypassed
    lin.set_lora_enabled(True)
    lin.write_lora(None, np.zeros_like(b))  # B = 0: PEFT-style init, exact no-op on the output
    assert rel_l2(lin.forward(x, m), base) < 2e-3
    lin.close()
    f.close()


def test_shape_errors_are_statuses(ctx):
    rng = np.random.default_rng(6)
    f = rt.Frozen.from_f32(ctx, (rng.standard_normal((64, 64)) * 0.02).astype(np.float32), Q.Q4_0)
    with pytest.raises(rt.RtError):
        rt.Linear("bad", f, np.zeros(3, np.float32))  # src/linear.rs:49-51 asserts bias length
    lin = rt.Linear("ok", f)
    with pytest.raises(rt.RtError):
        lin.attach_lora(8, 16.0, np.zeros((8, 32), np.float32), np.zeros((64, 8), np.float32))
    with pytest.raises(rt.RtError) as e:
        lin.attach_lora(65, 16.0, np.zeros((65, 64), np.float32), np.zeros((64, 65), np.float32))
    assert e.value.status == 7
    with pytest.raises(rt.RtError):
        lin.forward(np.zeros((2, 63), np.float32), 2)
    lin.close()
    f.close()
