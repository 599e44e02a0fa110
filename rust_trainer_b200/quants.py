"""NumPy encoders/decoders for the ggml block formats the frozen weights use.

Formats are the public ggml/GGUF ones (F16, BF16, Q8_0, Q4_0, Q4_K, Q6_K).  The encoders
exist so that synthetic GGUF-shaped models can be produced without a checkpoint (the
reference delegates this to rie-core's SyntheticSpec, src/main.rs:648-677); the decoders are
plain restatements of the block definitions and are what the tests compare the device's
`row()` against, next to the independent `gguf` package.

Every function works on a 2-D float32 matrix [rows, cols] <-> uint8 matrix [rows, row_bytes].
"""
from __future__ import annotations

import numpy as np

F16, Q4_0, Q8_0, Q4_K, Q6_K, BF16 = 1, 2, 8, 12, 14, 30
NAMES = {F16: "F16", Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", BF16: "BF16"}
BY_NAME = {v: k for k, v in NAMES.items()}
BLOCK = {F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), Q4_0: (32, 18), Q4_K: (256, 144), Q6_K: (256, 210)}


def row_bytes(t: int, cols: int) -> int:
    be, bb = BLOCK[t]
    if cols % be:
        raise ValueError(f"{NAMES[t]}: row length {cols} is not a multiple of {be}")
    return cols // be * bb


def _f16_bytes(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).view(np.uint8).reshape(*a.shape, 2)


def _rne(x: np.ndarray) -> np.ndarray:
    return np.rint(x)


# ----------------------------------------------------------------------------- encoders
def quantize(x: np.ndarray, t: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    if t == F16:
        return x.astype(np.float16).view(np.uint8).reshape(rows, cols * 2)
    if t == BF16:
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16  # round to nearest even
        return u.astype(np.uint16).view(np.uint8).reshape(rows, cols * 2)
    be, bb = BLOCK[t]
    if cols % be:
        raise ValueError(f"{NAMES[t]}: row length {cols} is not a multiple of {be}")
    nb = cols // be
    xb = x.reshape(rows, nb, be)
    out = np.zeros((rows, nb, bb), dtype=np.uint8)
    if t == Q8_0:
        amax = np.abs(xb).max(axis=2)
        df = (amax / np.float32(127.0)).astype(np.float32)  # ggml inverts the f32 scale, stores it as f16
        d = df.astype(np.float16)
        inv = np.where(df > 0, np.float32(1.0) / np.where(df > 0, df, 1), 0).astype(np.float32)
        v = xb * inv[..., None]
        q = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -127, 127).astype(np.int8)  # roundf
        out[..., 0:2] = _f16_bytes(d)
        out[..., 2:] = q.view(np.uint8)
    elif t == Q4_0:
        idx = np.abs(xb).argmax(axis=2)
        mx = np.take_along_axis(xb, idx[..., None], axis=2)[..., 0]
        df = (mx / np.float32(-8.0)).astype(np.float32)
        d = df.astype(np.float16)
        inv = np.where(df != 0, np.float32(1.0) / np.where(df != 0, df, 1), 0).astype(np.float32)
        q = np.clip(np.trunc(xb * inv[..., None] + np.float32(8.5)), 0, 15).astype(np.uint8)
        out[..., 0:2] = _f16_bytes(d)
        out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    elif t == Q4_K:
        sb = xb.reshape(rows, nb, 8, 32)
        mn = np.minimum(sb.min(axis=3), 0.0)
        mxv = sb.max(axis=3)
        scale = (mxv - mn) / 15.0
        minp = -mn
        d = (scale.max(axis=2) / 63.0).astype(np.float16)
        dmin = (minp.max(axis=2) / 63.0).astype(np.float16)
        df, dmf = d.astype(np.float32), dmin.astype(np.float32)
        sc = np.where(df[..., None] > 0, _rne(scale / np.where(df > 0, df, 1)[..., None]), 0).clip(0, 63).astype(np.uint8)
        m = np.where(dmf[..., None] > 0, _rne(minp / np.where(dmf > 0, dmf, 1)[..., None]), 0).clip(0, 63).astype(np.uint8)
        eff = df[..., None] * sc.astype(np.float32)
        off = dmf[..., None] * m.astype(np.float32)
        q = np.where(eff[..., None] > 0, _rne((sb + off[..., None]) / np.where(eff > 0, eff, 1)[..., None]), 0)
        q = q.clip(0, 15).astype(np.uint8)
        out[..., 0:2] = _f16_bytes(d)
        out[..., 2:4] = _f16_bytes(dmin)
        s12 = np.zeros((rows, nb, 12), dtype=np.uint8)
        s12[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
        s12[..., 4:8] = (m[..., 0:4] & 63) | ((m[..., 4:8] >> 4) << 6)
        s12[..., 8:12] = (sc[..., 4:8] & 15) | ((m[..., 4:8] & 15) << 4)
        out[..., 4:16] = s12
        qq = q.reshape(rows, nb, 4, 2, 32)
        out[..., 16:] = (qq[..., 0, :] | (qq[..., 1, :] << 4)).reshape(rows, nb, 128)
    elif t == Q6_K:
        sb = xb.reshape(rows, nb, 16, 16)
        amax = np.abs(sb).max(axis=3)
        scf = amax / 31.0
        d = (scf.max(axis=2) / 127.0).astype(np.float16)
        df = d.astype(np.float32)
        sc = np.where(df[..., None] > 0, _rne(scf / np.where(df > 0, df, 1)[..., None]), 0).clip(-128, 127).astype(np.int8)
        eff = df[..., None] * sc.astype(np.float32)
        q = np.where(eff[..., None] != 0, _rne(sb / np.where(eff != 0, eff, 1)[..., None]), 0).clip(-32, 31)
        q = (q + 32).astype(np.uint8).reshape(rows, nb, 2, 4, 32)  # [half, quarter, l]
        lo, hi = q & 15, q >> 4
        ql = np.zeros((rows, nb, 2, 64), dtype=np.uint8)
        ql[..., 0:32] = lo[..., 0, :] | (lo[..., 2, :] << 4)
        ql[..., 32:64] = lo[..., 1, :] | (lo[..., 3, :] << 4)
        qh = hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)
        out[..., 0:128] = ql.reshape(rows, nb, 128)
        out[..., 128:192] = qh.reshape(rows, nb, 64)
        out[..., 192:208] = sc.view(np.uint8)
        out[..., 208:210] = _f16_bytes(d)
    else:
        raise ValueError(f"unsupported ggml type {t}")
    return out.reshape(rows, nb * bb)


# ----------------------------------------------------------------------------- decoders
def dequantize(q: np.ndarray, t: int, cols: int) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    rows = q.shape[0]
    if t == F16:
        return q.view(np.float16).astype(np.float32).reshape(rows, cols)
    if t == BF16:
        return (q.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(rows, cols)
    be, bb = BLOCK[t]
    nb = cols // be
    b = q.reshape(rows, nb, bb)
    f16 = lambda a: np.ascontiguousarray(a).view(np.float16).astype(np.float32)[..., 0]
    if t == Q8_0:
        d = f16(b[..., 0:2])
        return (b[..., 2:].view(np.int8).astype(np.float32) * d[..., None]).reshape(rows, cols)
    if t == Q4_0:
        d = f16(b[..., 0:2])
        qs = b[..., 2:]
        v = np.concatenate([qs & 15, qs >> 4], axis=2).astype(np.float32) - 8.0
        return (v * d[..., None]).reshape(rows, cols)
    if t == Q4_K:
        d, dmin = f16(b[..., 0:2]), f16(b[..., 2:4])
        s = b[..., 4:16]
        sc = np.concatenate([s[..., 0:4] & 63, (s[..., 8:12] & 15) | ((s[..., 0:4] >> 6) << 4)], axis=2)
        m = np.concatenate([s[..., 4:8] & 63, (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)], axis=2)
        qs = b[..., 16:].reshape(rows, nb, 4, 32)
        codes = np.stack([qs & 15, qs >> 4], axis=3).reshape(rows, nb, 8, 32).astype(np.float32)
        dl = (d[..., None] * sc.astype(np.float32))[..., None]
        ml = (dmin[..., None] * m.astype(np.float32))[..., None]
        return (dl * codes - ml).reshape(rows, cols)
    if t == Q6_K:
        ql = b[..., 0:128].reshape(rows, nb, 2, 64)
        qh = b[..., 128:192].reshape(rows, nb, 2, 32)
        sc = b[..., 192:208].view(np.int8).astype(np.float32)
        d = f16(b[..., 208:210])
        lo = np.stack([ql[..., 0:32] & 15, ql[..., 32:64] & 15, ql[..., 0:32] >> 4, ql[..., 32:64] >> 4], axis=3)
        hi = np.stack([(qh >> (2 * i)) & 3 for i in range(4)], axis=3)
        codes = ((lo | (hi << 4)).astype(np.int8) - 32).astype(np.float32).reshape(rows, nb, 16, 16)
        eff = (d[..., None] * sc)[..., None]
        return (eff * codes).reshape(rows, cols)
    raise ValueError(f"unsupported ggml type {t}")
