"""Regenerates the committed fixtures in this directory.

  blocks_<FMT>.npz : ggml block bytes of a seeded 6 x 512 matrix and their f32 decode by the
                     independent `gguf` package (gguf.quants.dequantize), which implements the
                     public ggml formats the reference's rie-core dependency also implements.
  tiny_model.npz   : per-target log-probabilities, LoRA gradients and the adapter after three
                     AdamW steps of the CPU oracle on a seeded tiny Qwen3-shaped Q4_0 model.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))


def blocks():
    from gguf import GGMLQuantizationType as T
    from gguf import quants as gq

    from rust_trainer_b200 import quants as Q

    rng = np.random.default_rng(20240607)
    x = (rng.standard_normal((6, 512)) * 0.05).astype(np.float32)
    x[0, :32] = 0.0  # an all-zero block
    x[1, 5] = 3.0    # an outlier
    for t, gt in [(Q.F16, T.F16), (Q.BF16, T.BF16), (Q.Q8_0, T.Q8_0), (Q.Q4_0, T.Q4_0), (Q.Q4_K, T.Q4_K), (Q.Q6_K, T.Q6_K)]:
        packed = Q.quantize(x, t)
        src = packed.view(np.float16) if t == Q.F16 else packed
        ref = np.asarray(gq.dequantize(src, gt), dtype=np.float32).reshape(6, 512)
        np.savez_compressed(os.path.join(HERE, f"blocks_{Q.NAMES[t]}.npz"), packed=packed, decoded=ref, ggml_type=t)


def tiny_model_case():
    from rust_trainer_b200 import synth

    spec = synth.preset("tiny-qwen3", quant="Q4_0", seed=11, w_std=0.05)
    tensors = synth.build_tensors(spec)
    synth.perturb_norms(tensors, 12)
    adapters = synth.lora_adapters(spec, 8, 16.0, seed=13, b_std=0.02)
    toks = synth.token_batch(spec, 2, 48, 14)
    return spec, tensors, adapters, toks


def tiny_model():
    from oracle import oracle as O
    from rust_trainer_b200 import synth

    spec, tensors, adapters, toks = tiny_model_case()
    om = O.OracleModel(spec.config(), tensors)
    om.attach_lora(adapters)
    w_all, lps = 1.0 / (2 * 24), []
    state = {}
    out = {}
    for step in range(3):
        om.zero_grad()
        lps = []
        for s in range(2):
            tp, tt = synth.answer_targets(toks[s], 24)
            lp, _ = om.forward_backward(toks[s], tp, tt, np.full(tp.size, w_all, np.float32))
            lps.append(lp)
        if step == 0:
            out["logp"] = np.concatenate(lps)
            out["grads"] = np.concatenate([np.concatenate([e["ga"].ravel(), e["gb"].ravel()]) for e in om.lora])
        om.clip_grad_norm(1.0)
        om.adamw_step(state, 1e-3, wd=0.01)
    out["adapter_after_3"] = np.concatenate([np.concatenate([e["a"].ravel(), e["b"].ravel()]) for e in om.lora])
    np.savez_compressed(os.path.join(HERE, "tiny_model.npz"), **out)


if __name__ == "__main__":
    blocks()
    tiny_model()
    print("fixtures written to", HERE)
