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

    def close(self) -> None:
        if self._h:
            lib().rt_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):  # best effort
        try:
            self.close()
        except Exception:
            pass


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
