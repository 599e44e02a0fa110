"""The allocation-free form of backward_input against the ordinary device entry point.

Some hosts cannot let a library call cudaMalloc while they run (all of HBM belongs to their own
pool, or they sit in a loop that must not block on the driver's allocator).  For them
rt_frozen_backward_input_dev_noalloc keeps the partial sums of a long contraction in a fixed array
inside the library instead of grow-on-demand scratch.  The shape below is accumulated in pieces
(more than 16384 weight rows to contract), so the array is really used; both entry points run the same
kernel, so the results must agree to the last bit.  Two calls in a row check that the second
call is not disturbed by what the first left in the shared array.  Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

import rust_trainer_b200 as rt
from rust_trainer_b200 import quants as Q
from rust_trainer_b200._lib import DT_F16, DT_F32, lib

pytestmark = pytest.mark.gpu


def test_no_alloc_matches_regular_entry_point_twice(ctx):
    import torch

    L = lib()
    rng = np.random.default_rng(42)
    n, k = 32768, 256  # contraction over 32768 weight rows: four pieces of 8192 whose partial sums are added
    f = rt.Frozen.from_f32(ctx, (rng.standard_normal((n, k)) * 0.02).astype(np.float32), Q.Q8_0)
    for call, t in enumerate((200, 77)):
        dy = torch.randn(t, n, device="cuda", dtype=torch.float16)
        want = torch.full((t, k), float("nan"), device="cuda", dtype=torch.float32)
        got = torch.full((t, k), float("nan"), device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        ctx.check(L.rt_frozen_backward_input_dev(f._h, dy.data_ptr(), DT_F16, t, want.data_ptr(), DT_F32, 0))
        st = L.rt_frozen_backward_input_dev_noalloc(f._h, dy.data_ptr(), DT_F16, t, got.data_ptr(), DT_F32, 0)
        assert st == 0, (call, st)
        ctx.synchronize()
        a, b = want.cpu().numpy(), got.cpu().numpy()
        assert np.isfinite(a).all() and np.isfinite(b).all()
        assert np.array_equal(a, b), (call, float(np.abs(a - b).max()))
    # accumulate form on the second shape: dx += dy.W
    t = 77
    dy = torch.randn(t, n, device="cuda", dtype=torch.float16)
    base = torch.randn(t, k, device="cuda", dtype=torch.float32)
    want, got = base.clone(), base.clone()
    torch.cuda.synchronize()
    ctx.check(L.rt_frozen_backward_input_dev(f._h, dy.data_ptr(), DT_F16, t, want.data_ptr(), DT_F32, 1))
    assert L.rt_frozen_backward_input_dev_noalloc(f._h, dy.data_ptr(), DT_F16, t, got.data_ptr(), DT_F32, 1) == 0
    ctx.synchronize()
    assert np.array_equal(want.cpu().numpy(), got.cpu().numpy())
    f.close()


def test_no_alloc_refuses_more_than_its_array_holds(ctx):
    import torch

    L = lib()
    rng = np.random.default_rng(43)
    # 32768 weight rows to contract in four pieces, 2304 rows: 4 x 2304 x 256 floats = 2.25 Mi floats
    # of partial sums, more than the 2 Mi the array holds
    n, k, t = 32768, 256, 2304
    f = rt.Frozen.from_f32(ctx, (rng.standard_normal((n, k)) * 0.02).astype(np.float32), Q.Q8_0)
    dy = torch.zeros(t, n, device="cuda", dtype=torch.float16)
    dx = torch.zeros(t, k, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    assert L.rt_frozen_backward_input_dev_noalloc(f._h, dy.data_ptr(), DT_F16, t, dx.data_ptr(), DT_F32, 0) == 8  # RT_ERR_TOO_LARGE
    ctx.check(L.rt_frozen_backward_input_dev(f._h, dy.data_ptr(), DT_F16, t, dx.data_ptr(), DT_F32, 0))  # the ordinary call takes it
    assert L.rt_frozen_backward_input_dev_noalloc(f._h, dy.data_ptr(), DT_F16, 32, dx.data_ptr(), DT_F32, 0) == 0  # fewer rows fit
    assert L.rt_frozen_backward_input_dev_noalloc(f._h, dy.data_ptr(), 0, 32, dx.data_ptr(), DT_F32, 0) == 7  # f32 activations: bad argument
    ctx.synchronize()
    f.close()
