"""The trainer's two objectives as batch calls on the device model.

Mirrors `Trainer::example_grad` (src/train.rs:269-297) and `ensure_ref_logps` (src/train.rs:229-246):
the reference walks a batch one example at a time; gradients simply add over examples, so here a
whole batch is ONE `forward_backward` call with per-target weights.

* SFT: weight 1/batch_tokens on every answer target; loss = -sum(logp)/batch_tokens.
* DPO: reference log-probabilities with the adapters disabled (cached by the caller), then
  z = beta*((pc - rc) - (pr - rr)), L = softplus(-z)/batch_n, and the gradient is one pass over
  [chosen | rejected] with constant weights +c on the chosen targets, -c on the rejected ones,
  c = beta*sigmoid(-z)/batch_n  (dL/dpc = -c, dL/dpr = +c; `forward_backward` accumulates the
  gradient of -sum(w*logp), as the reference's does).
"""
from __future__ import annotations

import numpy as np

from .synth import answer_targets


def _layout(examples):
    """examples: [(tokens, answer_start)] -> sequences, global target positions/tokens, per-example slices."""
    seqs, tps, tts, spans, off, k = [], [], [], [], 0, 0
    for toks, answer_start in examples:
        toks = np.asarray(toks, dtype=np.int32)
        tp, tt = answer_targets(toks, answer_start)
        seqs.append(toks)
        tps.append(tp + off)
        tts.append(tt)
        spans.append((k, k + tp.size))
        off += toks.size
        k += tp.size
    return seqs, np.concatenate(tps), np.concatenate(tts), spans


def softplus(x: float) -> float:
    """src/tensor.rs:146-153 (threshold 20, as torch)."""
    x = np.float32(x)
    return float(x) if x > 20.0 else float(np.log1p(np.exp(x, dtype=np.float32), dtype=np.float32))


def sigmoid(x: float) -> float:
    return float(np.float32(1.0) / (np.float32(1.0) + np.exp(-np.float32(x), dtype=np.float32)))


def sum_logps(model, examples) -> np.ndarray:
    """sum_logp (src/train.rs:178-180) of every example, one forward-only call."""
    seqs, tp, tt, spans = _layout(examples)
    lp = model.score(seqs, tp, tt)[0]
    return np.array([lp[a:b].sum(dtype=np.float32) for a, b in spans], dtype=np.float32)


def sft_batch_grad(model, examples) -> float:
    """Accumulates the batch's gradient; returns its loss (src/train.rs:330, 271-277)."""
    seqs, tp, tt, _ = _layout(examples)
    batch_tokens = tp.size
    w = np.full(batch_tokens, 1.0 / batch_tokens, np.float32)
    lp, _ = model.forward_backward(seqs, tp, tt, w)
    return float(-lp.sum(dtype=np.float32) / np.float32(batch_tokens))


def dpo_ref_logps(model, pairs):
    """[(chosen, rejected)] of (tokens, answer_start) -> [(rc, rr)] with the adapters off (src/train.rs:229-246)."""
    model.set_lora_enabled(False)
    try:
        rc = sum_logps(model, [p[0] for p in pairs])
        rr = sum_logps(model, [p[1] for p in pairs])
    finally:
        model.set_lora_enabled(True)
    return list(zip(rc.tolist(), rr.tolist()))


def dpo_batch_grad(model, pairs, ref_logps, beta: float) -> float:
    """Accumulates the DPO gradient of a batch of preference pairs; returns the batch loss (src/train.rs:279-295)."""
    n = len(pairs)
    pc = sum_logps(model, [p[0] for p in pairs])
    pr = sum_logps(model, [p[1] for p in pairs])
    examples, coefs, loss = [], [], 0.0
    for i, (chosen, rejected) in enumerate(pairs):
        rc, rr = ref_logps[i]
        z = np.float32(beta) * ((pc[i] - np.float32(rc)) - (pr[i] - np.float32(rr)))
        c = np.float32(beta) * np.float32(sigmoid(-z)) / np.float32(n)
        examples += [chosen, rejected]
        coefs += [c, -c]
        loss += softplus(-z) / n
    seqs, tp, tt, spans = _layout(examples)
    w = np.empty(tp.size, np.float32)
    for (a, b), c in zip(spans, coefs):
        w[a:b] = c
    model.forward_backward(seqs, tp, tt, w)
    return float(loss)
