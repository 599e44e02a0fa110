"""Host-side mirror of `struct Model` and the optimiser step (reference src/model.rs:292-687,
src/optim.rs, src/train.rs:316-381) over the level-3 C ABI."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from ._lib import ModelConfig, RtError, lib
from .frozen import Context, _fp
from .linear import Linear

_I32P = C.POINTER(C.c_int32)


def _ip(a: np.ndarray):
    return a.ctypes.data_as(_I32P)


class Model:
    def __init__(self, ctx: Context, cfg: dict, tensors: dict, head_rows: int = 0):
        """cfg: keys of synth.ModelSpec.config(); tensors: GGUF name -> (ggml_type|0, rows, cols, ndarray)."""
        self.ctx = ctx
        self.cfg = dict(cfg)
        mc = ModelConfig(vocab=cfg["vocab"], hidden=cfg["hidden"], ff=cfg["ff"], n_layers=cfg["n_layers"],
                         n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"],
                         rot_dim=cfg["rot_dim"], rope_theta=cfg["rope_theta"],
                         rope_freq_scale=cfg.get("rope_freq_scale", 1.0), rms_eps=cfg["rms_eps"],
                         rope_neox=int(cfg["rope_neox"]), qk_norm=int(cfg["qk_norm"]),
                         tie_embeddings=int(cfg["tie_embeddings"]), head_rows=head_rows)
        self._h = C.c_void_p()
        ctx.check(lib().rt_model_create(ctx._h, C.byref(mc), C.byref(self._h)))
        # weights before their biases
        for name in sorted(tensors, key=lambda n: n.endswith(".bias")):
            t, rows, cols, arr = tensors[name]
            arr = np.ascontiguousarray(arr)
            ctx.check(lib().rt_model_set_tensor(self._h, name.encode(), int(t), rows, cols,
                                                arr.ctypes.data_as(C.c_void_p), arr.nbytes))
        ctx.check(lib().rt_model_finalize(self._h))

    # --- adapters
    def attach_lora(self, rank: int, alpha: float, targets: list | None = None, seed: int = 1234) -> int:
        self.lora_alpha = float(alpha)
        n = C.c_size_t()
        csv = None if targets is None else ",".join(targets).encode()
        self.ctx.check(lib().rt_model_attach_lora(self._h, rank, alpha, csv, seed, C.byref(n)))
        return n.value

    def lora_linears(self) -> list:
        out = []
        for i in range(lib().rt_model_num_lora(self._h)):
            h = lib().rt_model_lora_linear(self._h, i)
            out.append(Linear(lib().rt_linear_name(h).decode(), None, _handle=h, _ctx=self.ctx))
        return out

    def linear_shapes(self) -> list:
        """(GGUF module name, in_dim, out_dim) of every block's seven projections, in
        Block::linears order (src/model.rs:199-218), whether adapted or not."""
        c = self.cfg
        d, q, kv, ff = c["hidden"], c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"], c["ff"]
        dims = [("attn_q", d, q), ("attn_k", d, kv), ("attn_v", d, kv), ("attn_output", q, d),
                ("ffn_gate", d, ff), ("ffn_up", d, ff), ("ffn_down", ff, d)]
        return [(f"blk.{li}.{nm}", i, o) for li in range(c["n_layers"]) for nm, i, o in dims]

    def load_adapters(self, adapters: list) -> None:
        """Overwrites A and B of every adapter (same order as lora_linears())."""
        lins = self.lora_linears()
        if len(lins) != len(adapters):
            raise RtError(1, "adapter count mismatch")
        for lin, ad in zip(lins, adapters):
            lin.write_lora(ad["a"], ad["b"])

    def set_lora_enabled(self, on: bool) -> None:
        self.ctx.check(lib().rt_model_set_lora_enabled(self._h, int(on)))

    def zero_grad(self) -> None:
        self.ctx.check(lib().rt_model_zero_grad(self._h))

    def set_checkpointing(self, mode: int) -> None:
        """Model.checkpointing (src/model.rs:299): 1 = recompute each block before its backward,
        0 = keep every block's caches, -1 = keep them when they fit in device memory."""
        self.ctx.check(lib().rt_model_set_checkpointing(self._h, int(mode)))

    @property
    def checkpointing(self) -> bool:
        """The mode the last staged batch used."""
        return bool(lib().rt_model_checkpointing(self._h))

    def trainable_params(self) -> int:
        return self.grad_buffer()[1]

    def grad_buffer(self):
        p, n = C.c_void_p(), C.c_size_t()
        self.ctx.check(lib().rt_model_grad_buffer(self._h, C.byref(p), C.byref(n)))
        return p.value, n.value

    # --- passes
    @staticmethod
    def _batch(seqs):
        toks = np.ascontiguousarray(np.concatenate([np.asarray(s, dtype=np.int32).reshape(-1) for s in seqs]))
        offs = np.zeros(len(seqs) + 1, dtype=np.int32)
        offs[1:] = np.cumsum([np.asarray(s).size for s in seqs])
        return toks, offs

    def forward_backward(self, seqs, target_pos, target_tok, weights):
        """seqs: list of token arrays; target_pos are GLOBAL positions in the concatenation."""
        toks, offs = self._batch(seqs)
        tp = np.ascontiguousarray(target_pos, dtype=np.int32)
        tt = np.ascontiguousarray(target_tok, dtype=np.int32)
        w = np.ascontiguousarray(weights, dtype=np.float32)
        if not (tp.size == tt.size == w.size):
            raise RtError(1, "targets and weights differ in length")
        logp = np.empty(tp.size, dtype=np.float32)
        hits = C.c_int32()
        self.ctx.check(lib().rt_model_forward_backward(self._h, _ip(toks), _ip(offs), len(seqs), _ip(tp), _ip(tt), _fp(w),
                                                       tp.size, _fp(logp), C.byref(hits)))
        return logp, hits.value

    def _layout(self, groups):
        toks, offs = self._batch([g.tokens for g in groups])
        pos = np.ascontiguousarray(np.concatenate([g.positions for g in groups]), dtype=np.int32)
        seg = np.ascontiguousarray(np.concatenate([g.segments for g in groups]), dtype=np.int32)
        return toks, offs, pos, seg

    def forward_backward_packed(self, groups, target_pos, target_tok, weights):
        """Model::forward_backward_packed for a batch of packing.Packed groups laid end to end;
        target_pos index the concatenation of the groups' packed token arrays."""
        toks, offs, pos, seg = self._layout(groups)
        tp = np.ascontiguousarray(target_pos, dtype=np.int32)
        tt = np.ascontiguousarray(target_tok, dtype=np.int32)
        w = np.ascontiguousarray(weights, dtype=np.float32)
        if not (tp.size == tt.size == w.size):
            raise RtError(1, "targets and weights differ in length")
        logp = np.empty(tp.size, dtype=np.float32)
        hits = C.c_int32()
        self.ctx.check(lib().rt_model_forward_backward_layout(self._h, _ip(toks), _ip(offs), len(groups), _ip(pos), _ip(seg),
                                                              _ip(tp), _ip(tt), _fp(w), tp.size, _fp(logp), C.byref(hits)))
        return logp, hits.value

    def score_packed(self, groups, target_pos, target_tok):
        toks, offs, pos, seg = self._layout(groups)
        tp = np.ascontiguousarray(target_pos, dtype=np.int32)
        tt = np.ascontiguousarray(target_tok, dtype=np.int32)
        logp = np.empty(tp.size, dtype=np.float32)
        hits = C.c_int32()
        self.ctx.check(lib().rt_model_score_layout(self._h, _ip(toks), _ip(offs), len(groups), _ip(pos), _ip(seg), _ip(tp),
                                                   _ip(tt), tp.size, _fp(logp), C.byref(hits)))
        return logp, hits.value

    def score(self, seqs, target_pos, target_tok, want_logits: bool = False):
        toks, offs = self._batch(seqs)
        tp = np.ascontiguousarray(target_pos, dtype=np.int32)
        tt = np.ascontiguousarray(target_tok, dtype=np.int32)
        logp = np.empty(tp.size, dtype=np.float32)
        logits = np.empty((tp.size, self.cfg["vocab"]), dtype=np.float32) if want_logits else None
        hits = C.c_int32()
        self.ctx.check(lib().rt_model_score(self._h, _ip(toks), _ip(offs), len(seqs), _ip(tp), _ip(tt), tp.size, _fp(logp),
                                            C.byref(hits), None if logits is None else _fp(logits)))
        return logp, hits.value, logits

    def argmax_at(self, seqs, target_pos) -> np.ndarray:
        """Greedy token at each (global) position of a forward-only pass (src/eval.rs:162-167)."""
        toks, offs = self._batch(seqs)
        tp = np.ascontiguousarray(target_pos, dtype=np.int32)
        out = np.empty(tp.size, dtype=np.int32)
        self.ctx.check(lib().rt_model_argmax_layout(self._h, _ip(toks), _ip(offs), len(seqs), None, None, _ip(tp), tp.size,
                                                    _ip(out)))
        return out

    def argmax_at_packed(self, groups, target_pos) -> np.ndarray:
        toks, offs, pos, seg = self._layout(groups)
        tp = np.ascontiguousarray(target_pos, dtype=np.int32)
        out = np.empty(tp.size, dtype=np.int32)
        self.ctx.check(lib().rt_model_argmax_layout(self._h, _ip(toks), _ip(offs), len(groups), _ip(pos), _ip(seg), _ip(tp),
                                                    tp.size, _ip(out)))
        return out

    def allreduce_grads(self) -> None:
        """Sum of the flat LoRA-gradient buffer over the ranks of the context's communicator."""
        self.ctx.check(lib().rt_model_allreduce_grads(self._h))

    def optim_step(self, lr: float, max_norm: float = 1.0, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                   weight_decay: float = 0.0) -> float:
        """clip_grad_norm + AdamW::step; returns the pre-clip gradient norm."""
        norm = C.c_float()
        self.ctx.check(lib().rt_optim_step(self._h, lr, max_norm, beta1, beta2, eps, weight_decay, C.byref(norm)))
        return norm.value

    def optim_state(self):
        """(step count, flat Adam m, flat Adam v) in parameter order."""
        n = self.trainable_params()
        t = C.c_uint64()
        m, v = np.empty(n, np.float32), np.empty(n, np.float32)
        self.ctx.check(lib().rt_optim_state_read(self._h, C.byref(t), _fp(m), _fp(v)))
        return t.value, m, v

    def set_optim_state(self, t: int, m: np.ndarray, v: np.ndarray) -> None:
        m = np.ascontiguousarray(m, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        if m.size != self.trainable_params() or v.size != m.size:
            raise RtError(1, "optimizer state does not match parameters")  # src/optim.rs:57 asserts
        self.ctx.check(lib().rt_optim_state_write(self._h, int(t), _fp(m), _fp(v)))

    def close(self) -> None:
        if self._h:
            lib().rt_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def schedule_lr(peak: float, warmup: int, total: int, min_ratio: float, step: int) -> float:
    """Schedule::lr (reference src/optim.rs:102-111), f32 arithmetic."""
    f = np.float32
    if warmup > 0 and step < warmup:
        return float(f(peak) * f(step + 1) / f(warmup))
    span = max(total - warmup, 1) if total > warmup else 1
    p = min(f(step - min(warmup, step)) / f(span), f(1.0))
    cos = f(0.5) * (f(1.0) + f(math.cos(f(math.pi) * p)))
    return float(f(peak) * (f(min_ratio) + (f(1.0) - f(min_ratio)) * cos))
