"""Host-side mirror of the reference's frozen-weight plugin surface.

`Frozen` has the methods of `trait FrozenMatmul` (reference src/frozen.rs:14-25) with the same
names, argument meaning and error behaviour, over the C ABI.  Inputs and outputs are NumPy
float32 arrays in host memory, as the trait's `&[f32]` / `Vec<f32>` are.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import quants
from ._lib import OK, RtError, lib

_F32P = C.POINTER(C.c_float)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(_F32P)


class Context:
    """One per GPU (rt_ctx): device, stream and scratch memory."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        st = lib().rt_ctx_create(device, C.byref(self._h))
        if st != OK:
            raise RtError(st, f"rt_ctx_create(device={device}) failed; is a B200 (sm_100) visible?")
        self.device = device

    def check(self, st: int) -> None:
        if st != OK:
            raise RtError(st, lib().rt_last_error(self._h).decode())

    def synchronize(self) -> None:
        self.check(lib().rt_ctx_synchronize(self._h))

    @property
    def stream(self) -> int:
        return lib().rt_ctx_stream(self._h) or 0

    # --- data parallelism: one NCCL communicator per context (rt_comm_*)
    @staticmethod
    def comm_unique_id() -> bytes:
        """128 bytes that rank 0 creates and every rank passes to comm_init_rank."""
        buf = (C.c_uint8 * 128)()
        st = lib().rt_comm_unique_id(buf, 128)
        if st != OK:
            raise RtError(st, "rt_comm_unique_id failed (is libnccl.so.2 loadable?)")
        return bytes(buf)

    def comm_init_rank(self, nranks: int, rank: int, unique_id: bytes) -> None:
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        self.check(lib().rt_comm_init_rank(self._h, nranks, rank, buf, 128))

    def comm_size(self) -> int:
        return lib().rt_comm_size(self._h)

    def comm_allreduce_f32(self, dev_ptr: int, n: int) -> None:
        self.check(lib().rt_comm_allreduce_f32(self._h, C.c_void_p(dev_ptr), n))

    def close(self) -> None:
        if self._h:
            lib().rt_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):  # best effort
        try:
            self.close()
        except Exception:
            pass


def quantize_q8_0_f32scale(w: np.ndarray):
    """The trainer's own Q8_0 quantiser (src/frozen.rs:55-73), f32 arithmetic: scales
    [rows*cols/32] f32 and codes [rows*cols] int8.  `f32::round` rounds half away from zero."""
    blk = np.ascontiguousarray(w, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(blk).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    v = blk * inv[:, None]
    r = np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))
    return d, np.clip(r, -127, 127).astype(np.int8).reshape(-1)


class Frozen:
    """A frozen [out x in] weight in a ggml block format, resident on one GPU."""

    def __init__(self, ctx: Context, ggml_type: int, rows: int, cols: int, packed: np.ndarray):
        packed = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
        self.ctx = ctx
        self._h = C.c_void_p()
        st = lib().rt_frozen_create(ctx._h, int(ggml_type), rows, cols, packed.ctypes.data_as(C.c_void_p),
                                    packed.size, C.byref(self._h))
        ctx.check(st)
        self.ggml_type = int(ggml_type)

    @classmethod
    def from_f32(cls, ctx: Context, w: np.ndarray, ggml_type: int) -> "Frozen":
        """Quantises a float matrix to `ggml_type` on the host and uploads the blocks."""
        rows, cols = w.shape
        return cls(ctx, ggml_type, rows, cols, quants.quantize(w, ggml_type))

    @classmethod
    def f32(cls, ctx: Context, w: np.ndarray) -> "Frozen":
        """FrozenWeight::f32 (src/frozen.rs:49-52): an unquantised [out x in] matrix."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        if w.ndim != 2:
            raise RtError(1, "weight shape mismatch")
        return cls(ctx, 0, w.shape[0], w.shape[1], w)

    @classmethod
    def q8_0(cls, ctx: Context, w: np.ndarray) -> "Frozen":
        """FrozenWeight::q8_0 (src/frozen.rs:55-73): per 32 columns an f32 scale amax/127 and
        round(v/scale) clamped to +-127 as signed bytes; rows not a multiple of 32 long stay f32."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, cols = w.shape
        if cols % 32:
            return cls.f32(ctx, w)
        scales, qs = quantize_q8_0_f32scale(w)
        self = cls.__new__(cls)
        self.ctx = ctx
        self._h = C.c_void_p()
        ctx.check(lib().rt_frozen_create_q8_0(ctx._h, rows, cols, _fp(scales), qs.ctypes.data_as(C.POINTER(C.c_int8)),
                                              C.byref(self._h)))
        self.ggml_type = -8
        return self

    def out_dim(self) -> int:
        return lib().rt_frozen_out_dim(self._h)

    def in_dim(self) -> int:
        return lib().rt_frozen_in_dim(self._h)

    def nbytes(self) -> int:
        return lib().rt_frozen_nbytes(self._h)

    def forward(self, x: np.ndarray, t: int) -> np.ndarray:
        """y[t x out] = x[t x in] . W^T"""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size != t * self.in_dim():
            raise RtError(1, f"forward: x has {x.size} elements, expected {t}*{self.in_dim()}")
        y = np.empty((t, self.out_dim()), dtype=np.float32)
        self.ctx.check(lib().rt_frozen_forward(self._h, _fp(x), t, _fp(y)))
        return y

    def backward_input(self, dy: np.ndarray, t: int, dx: np.ndarray) -> None:
        """dx[t x in] += dy[t x out] . W   (accumulates, like the trait method)"""
        dy = np.ascontiguousarray(dy, dtype=np.float32)
        if dy.size != t * self.out_dim() or dx.size != t * self.in_dim():
            raise RtError(1, "backward_input: shape mismatch")
        if dx.dtype != np.float32 or not dx.flags.c_contiguous:
            raise RtError(7, "backward_input: dx must be a contiguous float32 array")
        self.ctx.check(lib().rt_frozen_backward_input(self._h, _fp(dy), t, _fp(dx)))

    def row(self, r: int) -> np.ndarray:
        out = np.empty(self.in_dim(), dtype=np.float32)
        if r < 0:
            raise RtError(6, "row index out of range")
        self.ctx.check(lib().rt_frozen_row(self._h, r, _fp(out)))
        return out

    def close(self) -> None:
        if self._h:
            lib().rt_frozen_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
