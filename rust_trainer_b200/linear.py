"""Host-side mirror of `struct Linear` / `struct Lora` (reference src/linear.rs:9-122)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import RtError, lib
from .frozen import Context, Frozen, _fp


class Linear:
    """Frozen weight + optional bias + optional LoRA adapter: y = W.x + b + (alpha/r).B.A.x"""

    def __init__(self, name: str, w: Frozen, bias: np.ndarray | None = None, _handle=None, _ctx=None):
        self.name = name
        self.w = w
        self.ctx: Context = _ctx if _ctx is not None else w.ctx
        self._owned = _handle is None
        if _handle is None:
            if bias is not None:
                bias = np.ascontiguousarray(bias, dtype=np.float32)
                if bias.size != w.out_dim():
                    raise RtError(1, f"{name}: bias has {bias.size} entries, expected {w.out_dim()}")
            self._h = C.c_void_p()
            self.ctx.check(lib().rt_linear_create(self.ctx._h, w._h, None if bias is None else _fp(bias),
                                                  name.encode(), C.byref(self._h)))
        else:
            self._h = C.c_void_p(_handle)

    def in_dim(self) -> int:
        return lib().rt_linear_in_dim(self._h)

    def out_dim(self) -> int:
        return lib().rt_linear_out_dim(self._h)

    @property
    def rank(self) -> int:
        return lib().rt_linear_lora_rank(self._h)

    def attach_lora(self, rank: int, alpha: float, a: np.ndarray, b: np.ndarray) -> None:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        if a.size != rank * self.in_dim() or b.size != self.out_dim() * rank:
            raise RtError(1, f"{self.name}: adapter shape mismatch")
        self.ctx.check(lib().rt_linear_attach_lora(self._h, rank, alpha, _fp(a), _fp(b)))

    def set_lora_enabled(self, on: bool) -> None:
        self.ctx.check(lib().rt_linear_set_lora_enabled(self._h, int(on)))

    def forward(self, x: np.ndarray, t: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size != t * self.in_dim():
            raise RtError(1, f"{self.name}: input shape")
        y = np.empty((t, self.out_dim()), dtype=np.float32)
        self.ctx.check(lib().rt_linear_forward(self._h, _fp(x), t, _fp(y)))
        return y

    def backward(self, x: np.ndarray, dy: np.ndarray, t: int) -> np.ndarray:
        """Accumulates the adapter gradients and returns dx (fresh)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        dy = np.ascontiguousarray(dy, dtype=np.float32)
        if x.size != t * self.in_dim() or dy.size != t * self.out_dim():
            raise RtError(1, f"{self.name}: backward shape")
        dx = np.empty((t, self.in_dim()), dtype=np.float32)
        self.ctx.check(lib().rt_linear_backward(self._h, _fp(x), _fp(dy), t, _fp(dx)))
        return dx

    def lora(self) -> dict:
        """Copies of a [r x in], b [out x r], ga, gb."""
        r = self.rank
        if r == 0:
            raise RtError(7, f"{self.name}: no adapter")
        a = np.empty((r, self.in_dim()), np.float32)
        b = np.empty((self.out_dim(), r), np.float32)
        ga, gb = np.empty_like(a), np.empty_like(b)
        self.ctx.check(lib().rt_lora_read(self._h, _fp(a), _fp(b), _fp(ga), _fp(gb)))
        return dict(a=a, b=b, ga=ga, gb=gb)

    def write_lora(self, a: np.ndarray | None, b: np.ndarray | None) -> None:
        a = None if a is None else np.ascontiguousarray(a, dtype=np.float32)
        b = None if b is None else np.ascontiguousarray(b, dtype=np.float32)
        self.ctx.check(lib().rt_lora_write(self._h, None if a is None else _fp(a), None if b is None else _fp(b)))

    def zero_grad(self) -> None:
        self.ctx.check(lib().rt_lora_zero_grad(self._h))

    def close(self) -> None:
        if self._owned and self._h:
            lib().rt_linear_destroy(self._h)
        self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
