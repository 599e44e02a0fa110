"""Host-side mirror of the per-row operations (reference src/ops.rs, src/tensor.rs) and of the
attention core (src/attention.rs) over the op-level C ABI: one device kernel per call, NumPy
float32 arrays in and out.  The training step does not come through here (it chains the same
kernels on the device); these calls are for checking one operation against the CPU path."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import RtError, lib
from .frozen import Context, _fp

_I32P = C.POINTER(C.c_int32)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _ip(a):
    return a.ctypes.data_as(_I32P)


def rmsnorm(ctx: Context, x, w, eps: float) -> np.ndarray:
    """ops.rs:8-35; x [rows x d]."""
    x, w = _f(x), _f(w)
    rows, d = x.shape
    if w.size != d:
        raise RtError(1, "rmsnorm: weight length")
    y = np.empty_like(x)
    ctx.check(lib().rt_op_rmsnorm(ctx._h, _fp(x), _fp(w), rows, d, eps, _fp(y)))
    return y


def rmsnorm_backward(ctx: Context, x, w, dy, eps: float) -> np.ndarray:
    """ops.rs:39-56."""
    x, w, dy = _f(x), _f(w), _f(dy)
    rows, d = x.shape
    dx = np.empty_like(x)
    ctx.check(lib().rt_op_rmsnorm_backward(ctx._h, _fp(x), _fp(w), _fp(dy), rows, d, eps, _fp(dx)))
    return dx


def _rope_args(positions, rot, neox, theta, freq_scale, factors):
    f = None if factors is None else _f(factors)
    return _i(positions), int(rot), int(bool(neox)), float(theta), float(freq_scale), f


def qk_norm_rope(ctx: Context, q_raw, k_raw, v_raw, positions, rot, neox, theta, freq_scale=1.0, factors=None,
                 q_norm_w=None, k_norm_w=None, eps=1e-6):
    """attention.rs:170-185 on q [M x nh x hd], k, v [M x nkv x hd]: QK-norm, RoPE, f16 rounding."""
    q_raw, k_raw, v_raw = _f(q_raw), _f(k_raw), _f(v_raw)
    M, nh, hd = q_raw.shape
    nkv = k_raw.shape[1]
    pos, rot, neox, theta, fs, f = _rope_args(positions, rot, neox, theta, freq_scale, factors)
    qw = None if q_norm_w is None else _f(q_norm_w)
    kw = None if k_norm_w is None else _f(k_norm_w)
    q, k, v = np.empty_like(q_raw), np.empty_like(k_raw), np.empty_like(v_raw)
    ctx.check(lib().rt_op_qk_norm_rope(ctx._h, _fp(q_raw), _fp(k_raw), _fp(v_raw), _ip(pos), M, nh, nkv, hd, rot, neox, theta,
                                       fs, None if f is None else _fp(f), 0 if f is None else f.size,
                                       None if qw is None else _fp(qw), None if kw is None else _fp(kw), eps,
                                       _fp(q), _fp(k), _fp(v)))
    return q, k, v


def qk_norm_rope_backward(ctx: Context, dq, dk, dv, q_raw, k_raw, positions, rot, neox, theta, freq_scale=1.0,
                          factors=None, q_norm_w=None, k_norm_w=None, eps=1e-6):
    """attention.rs:330-358: inverse rotation, then the norm's backward."""
    dq, dk, dv, q_raw, k_raw = _f(dq), _f(dk), _f(dv), _f(q_raw), _f(k_raw)
    M, nh, hd = q_raw.shape
    nkv = k_raw.shape[1]
    pos, rot, neox, theta, fs, f = _rope_args(positions, rot, neox, theta, freq_scale, factors)
    qw = None if q_norm_w is None else _f(q_norm_w)
    kw = None if k_norm_w is None else _f(k_norm_w)
    dq_raw, dk_raw, dv_out = np.empty_like(dq), np.empty_like(dk), np.empty_like(dv)
    ctx.check(lib().rt_op_qk_norm_rope_backward(ctx._h, _fp(dq), _fp(dk), _fp(dv), _fp(q_raw), _fp(k_raw), _ip(pos), M, nh,
                                                nkv, hd, rot, neox, theta, fs, None if f is None else _fp(f),
                                                0 if f is None else f.size, None if qw is None else _fp(qw),
                                                None if kw is None else _fp(kw), eps, _fp(dq_raw), _fp(dk_raw), _fp(dv_out)))
    return dq_raw, dk_raw, dv_out


def attention(ctx: Context, q, k, v, seq_start):
    """attention.rs:187-230; returns (o [M x nh x hd], lse [nh x M])."""
    q, k, v, ss = _f(q), _f(k), _f(v), _i(seq_start)
    M, nh, hd = q.shape
    nkv = k.shape[1]
    o = np.empty_like(q)
    lse = np.empty((nh, M), np.float32)
    ctx.check(lib().rt_op_attention(ctx._h, _fp(q), _fp(k), _fp(v), _ip(ss), M, nh, nkv, hd, _fp(o), _fp(lse)))
    return o, lse


def attention_backward(ctx: Context, q, k, v, d_o, seq_start):
    """attention.rs:246-329; returns (dq, dk, dv)."""
    q, k, v, d_o, ss = _f(q), _f(k), _f(v), _f(d_o), _i(seq_start)
    M, nh, hd = q.shape
    nkv = k.shape[1]
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    ctx.check(lib().rt_op_attention_backward(ctx._h, _fp(q), _fp(k), _fp(v), _fp(d_o), _ip(ss), M, nh, nkv, hd, _fp(dq),
                                             _fp(dk), _fp(dv)))
    return dq, dk, dv


def swiglu(ctx: Context, gate, up) -> np.ndarray:
    gate, up = _f(gate), _f(up)
    rows, ff = gate.shape
    h = np.empty_like(gate)
    ctx.check(lib().rt_op_swiglu(ctx._h, _fp(gate), _fp(up), rows, ff, _fp(h)))
    return h


def swiglu_backward(ctx: Context, gate, up, dh):
    gate, up, dh = _f(gate), _f(up), _f(dh)
    rows, ff = gate.shape
    dg, du = np.empty_like(gate), np.empty_like(gate)
    ctx.check(lib().rt_op_swiglu_backward(ctx._h, _fp(gate), _fp(up), _fp(dh), rows, ff, _fp(dg), _fp(du)))
    return dg, du


def cross_entropy(ctx: Context, logits, target, weight=None, want_argmax=False, want_dlogits=False):
    """model.rs:579-596 per row; returns dict(logp, hits[, argmax][, dlogits])."""
    logits, target = _f(logits), _i(target)
    rows, v = logits.shape
    w = None if weight is None else _f(weight)
    logp = np.empty(rows, np.float32)
    hits = C.c_int32()
    am = np.empty(rows, np.int32) if want_argmax else None
    dl = np.empty_like(logits) if want_dlogits else None
    ctx.check(lib().rt_op_cross_entropy(ctx._h, _fp(logits), rows, v, _ip(target), None if w is None else _fp(w), _fp(logp),
                                        C.byref(hits), None if am is None else _ip(am), None if dl is None else _fp(dl)))
    out = dict(logp=logp, hits=hits.value)
    if am is not None:
        out["argmax"] = am
    if dl is not None:
        out["dlogits"] = dl
    return out
