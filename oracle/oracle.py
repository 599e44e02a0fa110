"""ctypes wrapper of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
It restates the reference's CPU algorithm (see oracle.c for file:line citations) and is the
thing the CUDA path is checked against, never a fallback for it.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "liboracle.so"
_lib = None

F32P = C.POINTER(C.c_float)
I32P = C.POINTER(C.c_int)


class _Rope(C.Structure):
    """struct orc_rope of oracle.c."""

    _fields_ = [("rot_dim", C.c_int), ("neox", C.c_int), ("t", C.c_int), ("cos", F32P), ("sin", F32P)]


def _host_tag() -> str:
    """Identifies the CPU the library was built for (-march=native code must not travel)."""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                import hashlib

                return hashlib.sha1(line.encode()).hexdigest()
    except OSError:
        pass
    return "unknown"


def build(force: bool = False) -> Path:
    src = _HERE / "oracle.c"
    tag_file = _HERE / "liboracle.host"
    tag = _host_tag()
    stale = (not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime
             or not tag_file.exists() or tag_file.read_text() != tag)
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True, capture_output=True)
        tag_file.write_text(tag)
    return _LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB))
        L.orc_round_f16.restype = C.c_float
        L.orc_round_f16.argtypes = [C.c_float]
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [C.c_int, C.c_int]
        L.orc_dequant_row.argtypes = [C.c_int, C.c_void_p, C.c_int, F32P]
        L.orc_softmax_row.restype = C.c_float
        L.orc_softmax_row.argtypes = [F32P, C.c_int, F32P]
        L.orc_schedule_lr.restype = C.c_float
        L.orc_schedule_lr.argtypes = [C.c_float, C.c_uint64, C.c_uint64, C.c_float, C.c_uint64]
        L.orc_clip_grad_norm.restype = C.c_float
        L.orc_clip_grad_norm.argtypes = [C.POINTER(F32P), C.POINTER(C.c_size_t), C.c_int, C.c_float]
        L.orc_adamw_step.argtypes = [F32P, F32P, F32P, F32P, C.c_size_t, C.c_int] + [C.c_float] * 5
        L.orc_rng_new.restype = C.c_uint64
        L.orc_rng_new.argtypes = [C.c_uint64]
        L.orc_rng_next_u64.restype = C.c_uint64
        L.orc_rng_next_u64.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_uniform.restype = C.c_float
        L.orc_rng_uniform.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_normal.restype = C.c_float
        L.orc_rng_normal.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_fill_normal.argtypes = [C.POINTER(C.c_uint64), F32P, C.c_size_t, C.c_float]
        L.orc_rng_fill_uniform_sym.argtypes = [C.POINTER(C.c_uint64), F32P, C.c_size_t, C.c_float]
        L.orc_model_new.restype = C.c_void_p
        L.orc_model_new.argtypes = [C.c_int] * 4 + [C.c_float]
        L.orc_model_free.argtypes = [C.c_void_p]
        L.orc_model_set_flags.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_model_set_embed.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_model_set_lm_head.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.orc_model_set_final_norm.argtypes = [C.c_void_p, F32P]
        L.orc_model_set_rope_factors.argtypes = [C.c_void_p, F32P, C.c_int]
        L.orc_model_set_attn.argtypes = [C.c_void_p] + [C.c_int] * 5 + [C.c_float] * 2 + [C.c_int] * 3 + [F32P] * 4
        L.orc_model_set_linear.argtypes = [C.c_void_p] + [C.c_int] * 5 + [C.c_void_p, F32P]
        L.orc_model_set_lora.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float] + [F32P] * 4
        L.orc_model_set_lora_enabled.argtypes = [C.c_void_p, C.c_int]
        L.orc_model_forward_backward.restype = C.c_int
        L.orc_model_forward_backward.argtypes = [C.c_void_p, I32P, C.c_int, I32P, I32P, I32P, F32P, C.c_int, F32P]
        L.orc_model_score.restype = C.c_int
        L.orc_model_score.argtypes = [C.c_void_p, I32P, C.c_int, I32P, I32P, I32P, C.c_int, F32P, F32P]
        L.orc_frozen_forward_raw.argtypes = [C.c_int] * 3 + [C.c_void_p, F32P, C.c_int, F32P]
        L.orc_frozen_backward_input_raw.argtypes = [C.c_int] * 3 + [C.c_void_p, F32P, C.c_int, F32P]
        L.orc_linear_forward_raw.argtypes = [C.c_int] * 3 + [C.c_void_p, F32P, C.c_int, C.c_float, F32P, F32P, F32P, C.c_int, F32P]
        L.orc_linear_backward_raw.argtypes = [C.c_int] * 3 + [C.c_void_p, C.c_int, C.c_float] + [F32P] * 6 + [C.c_int, F32P]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_act_int8.argtypes = [C.c_int]
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_rmsnorm.argtypes = [F32P, F32P, C.c_int, C.c_int, C.c_float, C.c_int, F32P, F32P]
        L.orc_rmsnorm_backward.argtypes = [F32P, F32P, F32P, F32P, C.c_int, C.c_int, F32P]
        L.orc_rope_init.argtypes = [C.POINTER(_Rope), I32P, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, F32P, C.c_int]
        L.orc_rope_free.argtypes = [C.POINTER(_Rope)]
        L.orc_rope_apply.argtypes = [C.POINTER(_Rope), F32P, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_attn_core_forward.argtypes = [F32P, F32P, F32P, C.c_int, C.c_int, C.c_int, C.c_int, I32P, F32P, F32P]
        L.orc_attn_core_backward.argtypes = [F32P] * 5 + [C.c_int] * 4 + [I32P] + [F32P] * 3
        L.orc_swiglu.argtypes = [F32P, F32P, C.c_size_t, F32P]
        L.orc_swiglu_backward.argtypes = [F32P, F32P, F32P, C.c_size_t, F32P, F32P]
        _lib = L
    return _lib


def fp(a):
    return None if a is None else a.ctypes.data_as(F32P)


def ip(a):
    return None if a is None else a.ctypes.data_as(I32P)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ----------------------------------------------------------------------------- small ops
def round_f16(x: float) -> float:
    return float(lib().orc_round_f16(float(x)))


def dequant_rows(ggml_type: int, packed: np.ndarray, rows: int, cols: int) -> np.ndarray:
    L = lib()
    packed = np.ascontiguousarray(packed).view(np.uint8).reshape(rows, -1)
    rb = L.orc_row_bytes(ggml_type, cols)
    assert packed.shape[1] == rb, (packed.shape, rb)
    out = np.empty((rows, cols), dtype=np.float32)
    for r in range(rows):
        L.orc_dequant_row(ggml_type, packed[r].ctypes.data_as(C.c_void_p), cols, fp(out[r]))
    return out


def frozen_forward(ggml_type, rows, cols, packed, x, t):
    x = _f32(x)
    y = np.empty((t, rows), dtype=np.float32)
    packed = np.ascontiguousarray(packed)
    lib().orc_frozen_forward_raw(ggml_type, rows, cols, packed.ctypes.data_as(C.c_void_p), fp(x), t, fp(y))
    return y


def frozen_backward_input(ggml_type, rows, cols, packed, dy, t, dx):
    dy = _f32(dy)
    packed = np.ascontiguousarray(packed)
    lib().orc_frozen_backward_input_raw(ggml_type, rows, cols, packed.ctypes.data_as(C.c_void_p), fp(dy), t, fp(dx))


def linear_forward(ggml_type, rows, cols, packed, bias, rank, alpha, a, b, x, t):
    x = _f32(x)
    y = np.empty((t, rows), dtype=np.float32)
    packed = np.ascontiguousarray(packed)
    lib().orc_linear_forward_raw(ggml_type, rows, cols, packed.ctypes.data_as(C.c_void_p), fp(bias), rank, alpha,
                                 fp(a), fp(b), fp(x), t, fp(y))
    return y


def linear_backward(ggml_type, rows, cols, packed, rank, alpha, a, b, ga, gb, x, dy, t):
    x, dy = _f32(x), _f32(dy)
    dx = np.empty((t, cols), dtype=np.float32)
    packed = np.ascontiguousarray(packed)
    lib().orc_linear_backward_raw(ggml_type, rows, cols, packed.ctypes.data_as(C.c_void_p), rank, alpha, fp(a), fp(b),
                                  fp(ga), fp(gb), fp(x), fp(dy), t, fp(dx))
    return dx


def schedule_lr(peak, warmup, total, min_ratio, step) -> float:
    return float(lib().orc_schedule_lr(peak, warmup, total, min_ratio, step))


def softmax_row(logits: np.ndarray):
    logits = _f32(logits)
    p = np.empty_like(logits)
    lse = lib().orc_softmax_row(fp(logits), logits.size, fp(p))
    return float(lse), p


def set_num_threads(n: int) -> int:
    """Worker threads of the oracle's row/head loops; returns the count in effect."""
    lib().orc_set_num_threads(int(n))
    return int(lib().orc_num_threads())


def set_act_int8(on: bool) -> None:
    """Mode (ii) of the oracle: round activations to 8 bits per block before every quantised
    forward matmul, as the engine does (src/rie.rs:77-80).  Process-wide; off by default."""
    lib().orc_set_act_int8(int(on))


def rmsnorm(x, w, eps, fused_scale=False):
    """ops.rs:8-35; returns (y, inv_rms per row)."""
    x, w = _f32(x), _f32(w)
    rows, d = x.shape
    y, inv = np.empty_like(x), np.empty(rows, np.float32)
    lib().orc_rmsnorm(fp(x), fp(w), rows, d, eps, int(fused_scale), fp(y), fp(inv))
    return y, inv


def rmsnorm_backward(x, w, inv, dy):
    x, w, inv, dy = _f32(x), _f32(w), _f32(inv), _f32(dy)
    rows, d = x.shape
    dx = np.empty_like(x)
    lib().orc_rmsnorm_backward(fp(x), fp(w), fp(inv), fp(dy), rows, d, fp(dx))
    return dx


def rope_apply(x, positions, rot_dim, neox, base, freq_scale=1.0, factors=None, inverse=False):
    """Rope::at_positions + Rope::apply (ops.rs:112-184) on x [t x heads x head_dim]; returns a copy."""
    x = _f32(x).copy()
    t, heads, hd = x.shape
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    f = None if factors is None else _f32(factors)
    r = _Rope()
    lib().orc_rope_init(C.byref(r), ip(pos), t, rot_dim, int(bool(neox)), base, freq_scale, fp(f), 0 if f is None else f.size)
    lib().orc_rope_apply(C.byref(r), fp(x), t, heads, hd, int(inverse))
    lib().orc_rope_free(C.byref(r))
    return x


def attn_core_forward(q, k, v, seq_start):
    """attention.rs:187-230; q [t x nh x hd], k, v [t x nkv x hd]; returns (o, probs [nh x t x t])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    t, nh, hd = q.shape
    nkv = k.shape[1]
    ss = np.ascontiguousarray(seq_start, dtype=np.int32)
    probs = np.zeros((nh, t, t), np.float32)
    o = np.zeros_like(q)
    lib().orc_attn_core_forward(fp(q), fp(k), fp(v), t, nh, nkv, hd, ip(ss), fp(probs), fp(o))
    return o, probs


def attn_core_backward(q, k, v, probs, d_o, seq_start):
    """attention.rs:246-329; returns (dq, dk, dv)."""
    q, k, v, probs, d_o = _f32(q), _f32(k), _f32(v), _f32(probs), _f32(d_o)
    t, nh, hd = q.shape
    nkv = k.shape[1]
    ss = np.ascontiguousarray(seq_start, dtype=np.int32)
    dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    lib().orc_attn_core_backward(fp(q), fp(k), fp(v), fp(probs), fp(d_o), t, nh, nkv, hd, ip(ss), fp(dq), fp(dk), fp(dv))
    return dq, dk, dv


def swiglu(g, u):
    g, u = _f32(g), _f32(u)
    h = np.empty_like(g)
    lib().orc_swiglu(fp(g), fp(u), g.size, fp(h))
    return h


def swiglu_backward(g, u, dh):
    g, u, dh = _f32(g), _f32(u), _f32(dh)
    dg, du = np.empty_like(g), np.empty_like(g)
    lib().orc_swiglu_backward(fp(g), fp(u), fp(dh), g.size, fp(dg), fp(du))
    return dg, du


class Rng:
    """tensor.rs:155-199 (SplitMix64, 24-bit uniform, Box-Muller)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(lib().orc_rng_new(seed))

    def next_u64(self) -> int:
        return int(lib().orc_rng_next_u64(C.byref(self.state)))

    def uniform(self) -> float:
        return float(lib().orc_rng_uniform(C.byref(self.state)))

    def normal(self) -> float:
        return float(lib().orc_rng_normal(C.byref(self.state)))

    def vec_normal(self, n: int, std: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().orc_rng_fill_normal(C.byref(self.state), fp(out), n, std)
        return out

    def vec_uniform_sym(self, n: int, bound: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().orc_rng_fill_uniform_sym(C.byref(self.state), fp(out), n, bound)
        return out


# ----------------------------------------------------------------------------- whole model
LINEARS = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]


class OracleModel:
    """The reference's Model (src/model.rs:292-301) over GGUF-named tensors.

    `cfg` is a dict with the keys of rust_trainer_b200.synth.ModelSpec.config();
    `tensors` maps GGUF tensor names to (ggml_type, rows, cols, ndarray of packed bytes or f32).
    LoRA state (a, b, ga, gb per adapted linear, in Block::linears order) lives in NumPy arrays
    owned by this object, so tests can read and write them directly.
    """

    def __init__(self, cfg: dict, tensors: dict):
        L = lib()
        self.cfg = dict(cfg)
        self.keep = []
        self.h = L.orc_model_new(cfg["vocab"], cfg["hidden"], cfg["ff"], cfg["n_layers"], cfg["rms_eps"])

        def packed(name):
            t = tensors[name]
            arr = np.ascontiguousarray(t[3])
            self.keep.append(arr)
            return t[0], t[1], t[2], arr

        def f32(name):
            if name not in tensors:
                return None
            arr = _f32(tensors[name][3]).reshape(-1)
            self.keep.append(arr)
            return arr

        ty, _, _, emb = packed("token_embd.weight")
        L.orc_model_set_embed(self.h, ty, emb.ctypes.data_as(C.c_void_p))
        if "output.weight" in tensors:
            ty, _, _, out = packed("output.weight")
            L.orc_model_set_lm_head(self.h, ty, out.ctypes.data_as(C.c_void_p))
        else:
            L.orc_model_set_lm_head(self.h, ty, emb.ctypes.data_as(C.c_void_p))
        L.orc_model_set_final_norm(self.h, fp(f32("output_norm.weight")))
        rf = f32("rope_freqs.weight")
        if rf is not None:
            L.orc_model_set_rope_factors(self.h, fp(rf), rf.size)
        for li in range(cfg["n_layers"]):
            p = f"blk.{li}."
            L.orc_model_set_attn(self.h, li, cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["rot_dim"],
                                 cfg["rope_theta"], cfg.get("rope_freq_scale", 1.0), int(cfg["qk_norm"]),
                                 int(cfg["rope_neox"]), int(cfg.get("kv_f16", True)),
                                 fp(f32(p + "attn_q_norm.weight")), fp(f32(p + "attn_k_norm.weight")),
                                 fp(f32(p + "attn_norm.weight")), fp(f32(p + "ffn_norm.weight")))
            for wi, nm in enumerate(LINEARS):
                ty, rows, cols, arr = packed(p + nm + ".weight")
                L.orc_model_set_linear(self.h, li, wi, ty, rows, cols, arr.ctypes.data_as(C.c_void_p), fp(f32(p + nm + ".bias")))
        self.lora = []  # list of dicts in parameter order

    def attach_lora(self, adapters: list):
        """adapters: list of dicts {layer, which, rank, alpha, a [r x in], b [out x r]} in parameter order."""
        L = lib()
        self.lora = []
        for ad in adapters:
            a, b = _f32(ad["a"]).copy(), _f32(ad["b"]).copy()
            ent = dict(layer=ad["layer"], which=ad["which"], rank=ad["rank"], alpha=float(ad["alpha"]), a=a, b=b,
                       ga=np.zeros_like(a), gb=np.zeros_like(b))
            self.lora.append(ent)
            L.orc_model_set_lora(self.h, ent["layer"], ent["which"], ent["rank"], ent["alpha"], fp(a), fp(b), fp(ent["ga"]), fp(ent["gb"]))

    def zero_grad(self):
        for e in self.lora:
            e["ga"][...] = 0
            e["gb"][...] = 0

    def set_flags(self, checkpointing=True, logits_chunk=64):
        lib().orc_model_set_flags(self.h, int(checkpointing), int(logits_chunk))

    def forward_backward(self, tokens, targets_pos, targets_tok, weights, seg_start=None):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        tp = np.ascontiguousarray(targets_pos, dtype=np.int32)
        tt = np.ascontiguousarray(targets_tok, dtype=np.int32)
        w = _f32(weights)
        ss = None if seg_start is None else np.ascontiguousarray(seg_start, dtype=np.int32)
        logp = np.empty(tp.size, dtype=np.float32)
        hits = lib().orc_model_forward_backward(self.h, ip(tokens), tokens.size, ip(ss), ip(tp), ip(tt), fp(w), tp.size, fp(logp))
        return logp, hits

    def score(self, tokens, targets_pos, targets_tok, seg_start=None, want_logits=False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        tp = np.ascontiguousarray(targets_pos, dtype=np.int32)
        tt = np.ascontiguousarray(targets_tok, dtype=np.int32)
        ss = None if seg_start is None else np.ascontiguousarray(seg_start, dtype=np.int32)
        logp = np.empty(tp.size, dtype=np.float32)
        logits = np.empty((tp.size, self.cfg["vocab"]), dtype=np.float32) if want_logits else None
        hits = lib().orc_model_score(self.h, ip(tokens), tokens.size, ip(ss), ip(tp), ip(tt), tp.size, fp(logp), fp(logits))
        return logp, hits, logits

    def clip_grad_norm(self, max_norm: float) -> float:
        arrs = []
        for e in self.lora:
            arrs += [e["ga"], e["gb"]]
        ptrs = (F32P * len(arrs))(*[fp(a) for a in arrs])
        sizes = (C.c_size_t * len(arrs))(*[a.size for a in arrs])
        return float(lib().orc_clip_grad_norm(ptrs, sizes, len(arrs), max_norm))

    def adamw_step(self, state: dict, lr: float, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0):
        """optim.rs:48-69; `state` holds t and per-tensor m, v (created on first use)."""
        if "m" not in state:
            state["t"] = 0
            state["m"] = [np.zeros_like(x) for e in self.lora for x in (e["a"], e["b"])]
            state["v"] = [np.zeros_like(x) for e in self.lora for x in (e["a"], e["b"])]
        state["t"] += 1
        i = 0
        for e in self.lora:
            for p, g in ((e["a"], e["ga"]), (e["b"], e["gb"])):
                lib().orc_adamw_step(fp(p), fp(g), fp(state["m"][i]), fp(state["v"][i]), p.size, state["t"], lr, beta1, beta2, eps, wd)
                i += 1

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
