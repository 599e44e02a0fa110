"""Synthetic GGUF-shaped models, LoRA adapters and token batches.

Stands in for `rust_trainer synth` (reference src/main.rs:648-677, which delegates to
rie-core's SyntheticSpec) and for real checkpoints / confirmed data, neither of which exists
offline.  Tensors carry GGUF names (`token_embd.weight`, `blk.N.attn_q.weight`, ...) and ggml
block bytes, so they feed the device library and the CPU oracle identically.

Generation rules (recorded in every result JSON through `ModelSpec.describe()`):
  * linear weights ~ N(0, w_std) (std), quantised to `quant`; a tensor whose row length is not
    a multiple of the K-quant super-block (256) falls back to `fallback_quant` (Q4_K at hidden
    896 is impossible for most tensors); norm weights 1.0; q/k/v biases ~ N(0, bias_std)
  * LoRA: A ~ N(0, a_std) with a_std = 1/r, B ~ N(0, 1e-3): the configs' "N(0, 1/r)" is read as
    a std, like their "N(0, 0.02)" for weights; drawn with the trainer's own SplitMix64 stream
  * llama3 rope_freqs: the published Llama-3.1 frequency-dependent divisor rule
    (factor, low/high frequency factors 1/4, original context 8192)
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field

import numpy as np

from . import quants
from .rng import Rng

LINEARS = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]


@dataclass
class ModelSpec:
    arch: str = "qwen3"
    n_layers: int = 2
    hidden: int = 64
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 16
    ff: int = 128
    vocab: int = 256
    qk_norm: bool = True
    attn_bias: bool = False
    tie_embeddings: bool = True
    rope_theta: float = 1e6
    rope_neox: bool = True
    rope_freq_scale: float = 1.0
    rope_llama3_factor: float = 0.0  # > 0: emit rope_freqs.weight by the llama3 rule
    rot: int = 0  # rotated elements per head (rope.dimension_count); 0 = the whole head
    rms_eps: float = 1e-6
    quant: str = "Q4_0"
    fallback_quant: str = "Q4_0"
    w_std: float = 0.02
    bias_std: float = 0.01
    seed: int = 0

    @property
    def rot_dim(self) -> int:
        return self.rot if self.rot > 0 else self.head_dim

    def config(self) -> dict:
        return dict(arch=self.arch, vocab=self.vocab, hidden=self.hidden, ff=self.ff, n_layers=self.n_layers,
                    n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, rot_dim=self.rot_dim,
                    rope_theta=self.rope_theta, rope_freq_scale=self.rope_freq_scale, rope_neox=self.rope_neox,
                    qk_norm=self.qk_norm, rms_eps=self.rms_eps, tie_embeddings=self.tie_embeddings,
                    attn_bias=self.attn_bias, kv_f16=True)

    def describe(self) -> dict:
        d = asdict(self)
        d["lora_init"] = "A~N(0, std=1/r), B~N(0, std=1e-3), SplitMix64+Box-Muller"
        return d

    def linear_shapes(self) -> dict:
        d, q, kv = self.hidden, self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return {"attn_q": (q, d), "attn_k": (kv, d), "attn_v": (kv, d), "attn_output": (d, q),
                "ffn_gate": (self.ff, d), "ffn_up": (self.ff, d), "ffn_down": (d, self.ff)}

    def quant_for(self, cols: int) -> int:
        t = quants.BY_NAME[self.quant]
        if cols % quants.BLOCK[t][0]:
            t = quants.BY_NAME[self.fallback_quant]
        return t

    def frozen_params_per_layer(self) -> int:
        return sum(r * c for r, c in self.linear_shapes().values())


PRESETS = {
    # Qwen3-0.6B shape
    "qwen3-0.6b": dict(arch="qwen3", n_layers=28, hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, ff=3072,
                       vocab=151936, qk_norm=True, tie_embeddings=True, rope_theta=1e6, rope_neox=True),
    # Qwen2.5-0.5B shape
    "qwen2.5-0.5b": dict(arch="qwen2", n_layers=24, hidden=896, n_heads=14, n_kv_heads=2, head_dim=64, ff=4864,
                         vocab=151936, qk_norm=False, attn_bias=True, tie_embeddings=True, rope_theta=1e6),
    # Llama-3.2-3B shape
    "llama-3.2-3b": dict(arch="llama", n_layers=28, hidden=3072, n_heads=24, n_kv_heads=8, head_dim=128, ff=8192,
                         vocab=128256, qk_norm=False, tie_embeddings=True, rope_theta=5e5, rope_neox=False,
                         rope_llama3_factor=32.0),
    # Qwen3-4B shape
    "qwen3-4b": dict(arch="qwen3", n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, ff=9728,
                     vocab=151936, qk_norm=True, tie_embeddings=False, rope_theta=1e6),
    # small shapes for tests (same code paths, seconds on the CPU oracle)
    "tiny-qwen3": dict(arch="qwen3", n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ff=256, vocab=512,
                       qk_norm=True, tie_embeddings=True),
    "tiny-qwen2": dict(arch="qwen2", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ff=512, vocab=640,
                       qk_norm=False, attn_bias=True, tie_embeddings=True),
    "tiny-llama": dict(arch="llama", n_layers=2, hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, ff=512, vocab=384,
                       qk_norm=False, tie_embeddings=False, rope_theta=5e5, rope_neox=False, rope_llama3_factor=32.0),
    # the 0.6B shape's head layout (128-wide heads, QK-norm, rotate-half), partial rotation, and
    # more heads than the register-resident RoPE kernels take
    "tiny-qwen3-hd128": dict(arch="qwen3", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ff=512,
                             vocab=512, qk_norm=True, tie_embeddings=True),
    "tiny-rot32": dict(arch="qwen3", n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ff=256, vocab=512,
                       qk_norm=True, tie_embeddings=True, rot=32),
    "tiny-manyheads": dict(arch="qwen3", n_layers=1, hidden=128, n_heads=60, n_kv_heads=6, head_dim=64, ff=256,
                           vocab=512, qk_norm=True, tie_embeddings=True),
}


def preset(name: str, **over) -> ModelSpec:
    kw = dict(PRESETS[name])
    kw.update(over)
    return ModelSpec(**kw)


def llama3_rope_factors(rot_dim: int, theta: float, factor: float, low: float = 1.0, high: float = 4.0,
                        orig_ctx: int = 8192) -> np.ndarray:
    out = np.empty(rot_dim // 2, dtype=np.float32)
    low_wl, high_wl = orig_ctx / low, orig_ctx / high
    for i in range(rot_dim // 2):
        freq = theta ** (-2.0 * i / rot_dim)
        wl = 2 * math.pi / freq
        if wl < high_wl:
            out[i] = 1.0
        elif wl > low_wl:
            out[i] = factor
        else:
            smooth = (orig_ctx / wl - low) / (high - low)
            out[i] = 1.0 / ((1 - smooth) / factor + smooth)
    return out


def build_tensors(spec: ModelSpec) -> dict:
    """name -> (ggml_type or 0 for f32, rows, cols, ndarray): packed uint8 rows, or float32."""
    rng = np.random.default_rng(spec.seed)
    T: dict = {}

    def quantised(name, rows, cols):
        t = spec.quant_for(cols)
        # draw in slabs to bound peak memory on the large-vocabulary tables
        parts = []
        step = max(1, (1 << 24) // cols)
        for r0 in range(0, rows, step):
            n = min(step, rows - r0)
            w = rng.standard_normal((n, cols), dtype=np.float32) * np.float32(spec.w_std)
            parts.append(quants.quantize(w, t))
        T[name] = (t, rows, cols, np.concatenate(parts, axis=0))

    def f32(name, arr):
        T[name] = (0, 1, arr.size, np.ascontiguousarray(arr, dtype=np.float32))

    quantised("token_embd.weight", spec.vocab, spec.hidden)
    if not spec.tie_embeddings:
        quantised("output.weight", spec.vocab, spec.hidden)
    f32("output_norm.weight", np.ones(spec.hidden))
    if spec.rope_llama3_factor > 0:
        f32("rope_freqs.weight", llama3_rope_factors(spec.rot_dim, spec.rope_theta, spec.rope_llama3_factor))
    shapes = spec.linear_shapes()
    for li in range(spec.n_layers):
        p = f"blk.{li}."
        f32(p + "attn_norm.weight", np.ones(spec.hidden))
        f32(p + "ffn_norm.weight", np.ones(spec.hidden))
        if spec.qk_norm:
            f32(p + "attn_q_norm.weight", np.ones(spec.head_dim))
            f32(p + "attn_k_norm.weight", np.ones(spec.head_dim))
        for nm in LINEARS:
            rows, cols = shapes[nm]
            quantised(p + nm + ".weight", rows, cols)
            if spec.attn_bias and nm in ("attn_q", "attn_k", "attn_v"):
                f32(p + nm + ".bias", rng.standard_normal(rows).astype(np.float32) * np.float32(spec.bias_std))
    return T


def perturb_norms(tensors: dict, seed: int, spread: float = 0.2) -> None:
    """Replaces the all-ones norm weights by 1 +- spread (tests want non-trivial norms)."""
    rng = np.random.default_rng(seed)
    for k, (t, r, c, a) in list(tensors.items()):
        if k.endswith("norm.weight"):
            tensors[k] = (t, r, c, (1.0 + rng.uniform(-spread, spread, a.shape)).astype(np.float32))


def lora_adapters(spec: ModelSpec, rank: int, alpha: float, seed: int, targets=None, a_std=None,
                  b_std: float = 1e-3) -> list:
    """Adapters in parameter order: block order x Block::linears order (reference
    src/model.rs:199-218, src/optim.rs:32-34)."""
    targets = LINEARS if targets is None else targets
    a_std = 1.0 / rank if a_std is None else a_std
    rng = Rng(seed)
    shapes = spec.linear_shapes()
    out = []
    for li in range(spec.n_layers):
        for wi, nm in enumerate(LINEARS):
            if nm not in targets:
                continue
            rows, cols = shapes[nm]
            a = rng.normal(rank * cols, a_std).reshape(rank, cols)
            b = rng.normal(rows * rank, b_std).reshape(rows, rank)
            out.append(dict(layer=li, which=wi, name=f"blk.{li}.{nm}", rank=rank, alpha=float(alpha), a=a, b=b))
    return out


def token_batch(spec: ModelSpec, n_seq: int, seq_len: int, seed: int) -> np.ndarray:
    """Uniform-random ids in [0, vocab): [n_seq, seq_len] int32."""
    return np.random.default_rng(seed).integers(0, spec.vocab, size=(n_seq, seq_len), dtype=np.int32)


def answer_targets(tokens: np.ndarray, answer_start: int):
    """model.rs:230-232: target i predicts tokens[i] from position i-1, i >= max(answer_start, 1)."""
    idx = np.arange(max(answer_start, 1), tokens.size)
    return (idx - 1).astype(np.int32), tokens[idx].astype(np.int32)
