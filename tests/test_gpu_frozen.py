"""FrozenMatmul on the GPU (through the C ABI) against the CPU oracle.

Mirrors the reference's own checks: backward_input equals the dense dy.W built from row()
(tests/engine.rs:96-120, tolerance 1e-3), the adjoint identity (src/frozen.rs:218-227), and
shape refusals (the reference panics; here a status).  Rows are bit exact (byte/integer
work); matmuls use f16 operands with f32 accumulation, tolerance 2e-3 relative L2.
"""
import numpy as np
import pytest

import rust_trainer_b200 as rt
from conftest import rel_l2
from oracle import oracle as O
from rust_trainer_b200 import quants as Q

pytestmark = pytest.mark.gpu

FORMATS = [Q.F16, Q.BF16, Q.Q8_0, Q.Q4_0, Q.Q4_K, Q.Q6_K]
MATMUL_TOL = 2e-3


def _shapes(t):
    pair = [(1024, 512, 2500), (512, 512, 5001)]  # enough 256-row tiles for the CTA-pair kernel
    if t in (Q.Q4_K, Q.Q6_K):
        return [(128, 256, 40), (384, 512, 300), (1024, 1024, 513)] + pair
    return [(128, 64, 1), (256, 128, 100), (192, 96, 7), (896, 896, 300), (1024, 1024, 513)] + pair


@pytest.mark.parametrize("t", FORMATS, ids=[Q.NAMES[t] for t in FORMATS])
def test_rows_are_bit_exact(ctx, t):
    rng = np.random.default_rng(t)
    n, k = 200, 512
    packed = Q.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), t)
    want = O.dequant_rows(t, packed, n, k)
    f = rt.Frozen(ctx, t, n, k, packed)
    assert (f.out_dim(), f.in_dim(), f.nbytes()) == (n, k, packed.size)
    for r in (0, 1, 63, 64, 127, 128, 199):
        assert np.array_equal(f.row(r), want[r]), r
    with pytest.raises(rt.RtError) as e:
        f.row(n)
    assert e.value.status == 6
    f.close()


@pytest.mark.parametrize("t", FORMATS, ids=[Q.NAMES[t] for t in FORMATS])
def test_forward_and_backward_input(ctx, t):
    rng = np.random.default_rng(100 + t)
    for n, k, m in _shapes(t):
        packed = Q.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), t)
        f = rt.Frozen(ctx, t, n, k, packed)
        x = rng.standard_normal((m, k)).astype(np.float32)
        assert rel_l2(f.forward(x, m), O.frozen_forward(t, n, k, packed, x, m)) < MATMUL_TOL, (n, k, m)
        dy = rng.standard_normal((m, n)).astype(np.float32)
        dx0 = rng.standard_normal((m, k)).astype(np.float32)
        dx, ref = dx0.copy(), dx0.copy()
        f.backward_input(dy, m, dx)  # accumulates, like the trait method
        O.frozen_backward_input(t, n, k, packed, dy, m, ref)
        assert rel_l2(dx, ref) < MATMUL_TOL, (n, k, m)
        f.close()


@pytest.mark.parametrize("t", [Q.Q8_0, Q.Q4_0, Q.Q6_K])
def test_adjoint_identity_on_device(ctx, t):
    rng = np.random.default_rng(7)
    n, k, m = 384, 512, 33
    f = rt.Frozen.from_f32(ctx, (rng.standard_normal((n, k)) * 0.1).astype(np.float32), t)
    x = rng.standard_normal((m, k)).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    y = f.forward(x, m)
    dx = np.zeros((m, k), np.float32)
    f.backward_input(dy, m, dx)
    lhs, rhs = float((dy.astype(np.float64) * y).sum()), float((dx.astype(np.float64) * x).sum())
    assert abs(lhs - rhs) <= 2e-3 * max(1.0, abs(lhs))
    f.close()


@pytest.mark.parametrize("n,k,tokens", [(512, 256, 300), (384, 256, 1000), (1024, 128, 4133)])
def test_16_bit_outputs_are_the_rounded_f32_outputs(ctx, n, k, tokens):
    """The device entry points write f32, f16 or bf16.  The 16-bit epilogue (fragment-layout TMEM
    loads, paired rounding, transposing matrix stores, swizzled TMA store) must give exactly the
    f32 result rounded once, for the CTA-pair kernel (a multiple of 256 features), the single-CTA
    one, and token counts that end inside a tile and inside a 32-token block."""
    import torch

    from rust_trainer_b200._lib import DT_BF16, DT_F16, DT_F32, lib

    L = lib()
    rng = np.random.default_rng(n + tokens)
    f = rt.Frozen.from_f32(ctx, (rng.standard_normal((n, k)) * 0.05).astype(np.float32), Q.Q8_0)
    x = torch.randn(tokens, k, device="cuda", dtype=torch.float16)
    y32 = torch.full((tokens, n), float("nan"), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    ctx.check(L.rt_frozen_forward_dev(f._h, x.data_ptr(), DT_F16, tokens, y32.data_ptr(), DT_F32, 0))
    for dt, tdt in ((DT_F16, torch.float16), (DT_BF16, torch.bfloat16)):
        y16 = torch.full((tokens + 1, n), 7.0, device="cuda", dtype=tdt)  # one guard row behind the output
        torch.cuda.synchronize()
        ctx.check(L.rt_frozen_forward_dev(f._h, x.data_ptr(), DT_F16, tokens, y16.data_ptr(), dt, 0))
        ctx.synchronize()
        assert torch.equal(y16[:tokens], y32.to(tdt)), (dt, float((y16[:tokens].float() - y32).abs().max()))
        assert bool((y16[tokens] == 7.0).all())  # nothing written past the last token
    f.close()


def test_empty_and_refused_inputs(ctx):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((64, 64)) * 0.02).astype(np.float32)
    f = rt.Frozen.from_f32(ctx, w, Q.Q4_0)
    assert f.forward(np.zeros((0, 64), np.float32), 0).shape == (0, 64)  # t = 0 is a no-op
    with pytest.raises(rt.RtError):
        f.forward(np.zeros((3, 32), np.float32), 3)  # wrong inner dimension
    f.close()
    packed = Q.quantize(w, Q.Q4_0)
    with pytest.raises(rt.RtError) as e:
        rt.Frozen(ctx, 3, 64, 64, packed)  # Q4_1: unsupported
    assert e.value.status == 2
    with pytest.raises(rt.RtError) as e:
        rt.Frozen(ctx, Q.Q4_0, 64, 64, packed[:-1])  # byte count does not match
    assert e.value.status == 1
    with pytest.raises(rt.RtError) as e:
        rt.Frozen(ctx, Q.Q4_K, 4, 128, np.zeros(4 * 72, np.uint8))  # 128 is not a multiple of 256
    assert e.value.status == 1


def test_full_size_properties(ctx):
    """The benchmark's sizes (ffn_gate of the 0.6B shape, 3072 x 1024, at 8192 tokens), checked by
    properties that do not need the oracle: linearity in x and the adjoint identity."""
    rng = np.random.default_rng(3)
    n, k, m = 3072, 1024, 8192
    f = rt.Frozen.from_f32(ctx, (rng.standard_normal((n, k)) * 0.02).astype(np.float32), Q.Q8_0)
    x1 = rng.standard_normal((m, k)).astype(np.float32)
    x2 = rng.standard_normal((m, k)).astype(np.float32)
    y1, y2, y12 = f.forward(x1, m), f.forward(x2, m), f.forward(x1 + x2, m)
    assert rel_l2(y12, y1 + y2) < MATMUL_TOL
    dy = rng.standard_normal((m, n)).astype(np.float32)
    dx = np.zeros((m, k), np.float32)
    f.backward_input(dy, m, dx)
    lhs, rhs = float((dy.astype(np.float64) * y1).sum()), float((dx.astype(np.float64) * x1).sum())
    assert abs(lhs - rhs) <= 2e-3 * abs(lhs) + 50.0  # inner products of ~2.5e7 random terms
    f.close()


def test_a_wait_that_runs_out_is_a_status_not_a_hang(ctx):
    """Every device-side wait is bounded: a barrier nothing arrives on makes the wait give up after
    its limit (here 2e8 cycles, about 0.1 s), the kernel returns, the host reads
    RT_ERR_DEVICE_WAIT_TIMEOUT with the wait's site code, and the context keeps working."""
    from rust_trainer_b200._lib import lib

    st = lib().rt_ctx_selftest_wait_timeout(ctx._h, 200_000_000)
    assert st == 5  # RT_ERR_DEVICE_WAIT_TIMEOUT
    assert b"site 999" in lib().rt_last_error(ctx._h)
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((128, 64)) * 0.02).astype(np.float32)
    f = rt.Frozen.from_f32(ctx, w, Q.Q8_0)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    assert rel_l2(f.forward(x, 5), x @ O.dequant_rows(Q.Q8_0, Q.quantize(w, Q.Q8_0), 128, 64).T) < MATMUL_TOL
    f.close()


def test_builtin_f32_and_q8_0_weights(ctx):
    """FrozenWeight::{F32, Q8_0} (src/frozen.rs:33-187) with the reference's own unit test
    (src/frozen.rs:206-228): Q8_0 forward within 0.02 of f32, and the adjoint identity
    <dy, x.W^T> == <dy.W, x> to 1e-3 for both storages; plus exact rows and the oracle."""
    r = O.Rng(3)
    out, inp, t = 8, 64, 3  # the reference's test has 6 rows; 16-bit operand rows must be a multiple of 8 long here
    w = r.vec_normal(out * inp, 0.1).reshape(out, inp)
    x = r.vec_normal(t * inp, 1.0).reshape(t, inp)
    dy = r.vec_normal(t * out, 1.0).reshape(t, out)
    f = rt.Frozen.f32(ctx, w)
    q = rt.Frozen.q8_0(ctx, w)
    assert f.nbytes() == out * inp * 4 and q.nbytes() == out * inp // 32 * 4 + out * inp  # src/frozen.rs:181-186
    yf, yq = f.forward(x, t), q.forward(x, t)
    assert np.max(np.abs(yf - yq)) < 0.02
    assert rel_l2(yf, x @ w.T) < 1e-3
    for wq in (f, q):
        y = wq.forward(x, t)
        dx = np.zeros((t, inp), np.float32)
        wq.backward_input(dy, t, dx)
        lhs, rhs = float((dy * y).sum()), float((dx * x).sum())
        assert abs(lhs - rhs) < 1e-3 * max(abs(lhs), 1.0)
    assert np.array_equal(f.row(4), w[4])
    from rust_trainer_b200.frozen import quantize_q8_0_f32scale

    d, qs = quantize_q8_0_f32scale(w)
    deq = (np.repeat(d, 32) * qs.astype(np.float32)).reshape(out, inp)
    assert np.array_equal(q.row(5), deq[5])
    f.close()
    q.close()
    # a wide f32 weight against the oracle's F32 rows, both directions
    rng = np.random.default_rng(9)
    n, k, m = 384, 1024, 300
    w2 = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x2 = rng.standard_normal((m, k)).astype(np.float32)
    dy2 = rng.standard_normal((m, n)).astype(np.float32)
    f2 = rt.Frozen.f32(ctx, w2)
    assert rel_l2(f2.forward(x2, m), O.frozen_forward(0, n, k, w2, x2, m)) < MATMUL_TOL
    dx, ref = np.zeros((m, k), np.float32), np.zeros((m, k), np.float32)
    f2.backward_input(dy2, m, dx)
    O.frozen_backward_input(0, n, k, w2, dy2, m, ref)
    assert rel_l2(dx, ref) < MATMUL_TOL
    f2.close()
