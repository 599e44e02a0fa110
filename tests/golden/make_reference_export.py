"""Pins the CPU oracle's whole-model numbers against the reference's own float64 checker.

The reference checks its trainer with an independent NumPy float64 decoder
(tools/reference_check.py) that reads one safetensors file written by
examples/export_reference.rs:79-125: the model's dequantised f32 weights, a LoRA adapter on
every projection, one example, and the trainer's loss and analytic LoRA gradients.  The Rust
half cannot run here (no Rust toolchain); this script plays its part with the ORACLE in the
trainer's seat: it builds a small smooth model the way the exporter does (weights replaced by
their exact f32 dequantisation, f16 K/V rounding off, adapters of rank 4 with scale 2 on all
seven projections, A ~ U(+-1/sqrt(in)) from Rng(7), B ~ 0.02 * normal from Rng(11), mean
weights over the answer span), runs `oracle.OracleModel.forward_backward`, and writes the
exporter's file layout.

  python tests/golden/make_reference_export.py OUT_DIR
      writes one export per model shape into OUT_DIR (what tests/test_reference_check.py feeds
      to the reference's checker when the reference tree is present)

  python tests/golden/make_reference_export.py --fixture REFERENCE_TOOLS_DIR
      additionally imports `Reference` from REFERENCE_TOOLS_DIR/reference_check.py and stores its
      float64 loss, directional finite differences and single-entry finite differences in
      tests/golden/reference_check_float64.npz, the fixture the test compares the oracle with on
      machines that do not have the reference tree.

What the checker cannot see (so these stay pinned only by the oracle's own finite-difference
tests): rope_freqs divisors, the f16 K/V rounding, per-target weights other than the mean.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))

# three shapes, one per family the reference reports on (README.md:201-205): QK-norm + tied
# (Qwen3), q/k/v bias + tied (Qwen2.5), interleaved RoPE pairs + untied head (Llama / SmolLM2)
SHAPES = {
    "qwen3": dict(preset="tiny-qwen3", over=dict(n_layers=3)),
    "qwen2": dict(preset="tiny-qwen2", over=dict(n_layers=3, hidden=128, ff=256)),
    "llama": dict(preset="tiny-llama", over=dict(n_layers=3, hidden=128, ff=256, head_dim=64, rope_llama3_factor=0.0)),
}
RANK, SEQ, ANSWER_START = 4, 48, 28


def smooth_case(name: str):
    """(cfg, f32 tensors, adapters, tokens) of one shape, built as export_reference.rs:30-65 does."""
    from oracle import oracle as O
    from rust_trainer_b200 import synth
    from rust_trainer_b200.rng import Rng

    sh = SHAPES[name]
    spec = synth.preset(sh["preset"], quant="Q4_0", seed=31, w_std=0.08, **sh["over"])
    tensors = synth.build_tensors(spec)
    synth.perturb_norms(tensors, 5)
    smooth = {}
    for k, (t, rows, cols, arr) in tensors.items():
        if t == 0:
            smooth[k] = (0, rows, cols, arr)
        else:  # "replaced by their exact f32 dequantisation"
            smooth[k] = (0, rows, cols, O.dequant_rows(t, arr, rows, cols))
    cfg = spec.config()
    cfg["kv_f16"] = False
    ra, rb = Rng(7), Rng(11)
    adapters = []
    shapes = spec.linear_shapes()
    for li in range(spec.n_layers):
        for wi, nm in enumerate(synth.LINEARS):
            rows, cols = shapes[nm]
            a = ra.uniform_sym(RANK * cols, 1.0 / np.sqrt(np.float32(cols))).reshape(RANK, cols)
            adapters.append(dict(layer=li, which=wi, name=f"blk.{li}.{nm}", rank=RANK, alpha=2.0 * RANK, a=a, b=None))
    for ad in adapters:  # the exporter draws every A first (attach_lora), then every B
        rows = shapes[ad["name"].split(".")[-1]][0]
        ad["b"] = (rb.normal(rows * RANK) * np.float32(0.02)).reshape(rows, RANK)
    tokens = np.random.default_rng(17).integers(0, spec.vocab, SEQ, dtype=np.int32)
    return spec, cfg, smooth, adapters, tokens


def oracle_run(cfg, smooth, adapters, tokens):
    from oracle import oracle as O
    from rust_trainer_b200 import synth

    om = O.OracleModel(cfg, smooth)
    om.attach_lora(adapters)
    om.zero_grad()
    tp, tt = synth.answer_targets(tokens, ANSWER_START)
    w = np.full(tp.size, 1.0 / tp.size, np.float32)
    lp, _ = om.forward_backward(tokens, tp, tt, w)
    loss = float(-np.sum(lp.astype(np.float64)) / tp.size)
    grads = [(e["ga"].copy(), e["gb"].copy()) for e in om.lora]
    om.close()
    return loss, grads


def write_export(path, spec, cfg, smooth, adapters, tokens, loss, grads):
    """The file layout of examples/export_reference.rs:79-125."""
    from safetensors.numpy import save_file

    out = {}
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    out["token_embd"] = f32(smooth["token_embd.weight"][3]).reshape(spec.vocab, spec.hidden)
    if not spec.tie_embeddings:
        out["output"] = f32(smooth["output.weight"][3]).reshape(spec.vocab, spec.hidden)
    out["output_norm"] = f32(smooth["output_norm.weight"][3]).reshape(-1)
    for k, (_, rows, cols, arr) in smooth.items():
        if not k.startswith("blk."):
            continue
        if k.endswith("norm.weight"):
            out[k[: -len(".weight")]] = f32(arr).reshape(-1)
        elif k.endswith(".bias"):
            out[k] = f32(arr).reshape(-1)
        else:
            out[k] = f32(arr).reshape(rows, cols)
    for ad, (ga, gb) in zip(adapters, grads):
        out[ad["name"] + ".lora_a"] = f32(ad["a"])
        out[ad["name"] + ".lora_b"] = f32(ad["b"])
        out[ad["name"] + ".grad_a"] = f32(ga)
        out[ad["name"] + ".grad_b"] = f32(gb)
    out["tokens"] = tokens.astype(np.float32)
    meta = dict(arch=spec.arch, n_layer=spec.n_layers, hidden=spec.hidden, vocab=spec.vocab, n_head=spec.n_heads,
                n_kv_head=spec.n_kv_heads, head_dim=spec.head_dim, rot_dim=spec.rot_dim, rope_theta=spec.rope_theta,
                rope_neox=bool(spec.rope_neox), rope_freq_scale=spec.rope_freq_scale, rms_eps=spec.rms_eps,
                tied=bool(spec.tie_embeddings), lora_scale=2.0, rank=RANK, answer_start=ANSWER_START, loss=loss,
                lora=[ad["name"] for ad in adapters])
    save_file(out, str(path), metadata={"reference": json.dumps(meta)})


def export(name: str, path) -> None:
    spec, cfg, smooth, adapters, tokens = smooth_case(name)
    loss, grads = oracle_run(cfg, smooth, adapters, tokens)
    write_export(path, spec, cfg, smooth, adapters, tokens, loss, grads)


def directions(d_i: int, shapes) -> dict:
    """Unit direction number d_i over every adapter weight: name -> [dA, dB].  Seeded, so the
    fixture stores only the finite difference along it and the test rebuilds the direction."""
    rng = np.random.default_rng(1000 + d_i)
    dirs = {n: [rng.standard_normal(sa), rng.standard_normal(sb)] for n, sa, sb in shapes}
    norm = np.sqrt(sum((x * x).sum() for pair in dirs.values() for x in pair))
    return {n: [a / norm, b / norm] for n, (a, b) in dirs.items()}


def float64_fixture(tools_dir: str, out_dir: str) -> None:
    """Runs the reference's float64 decoder on each export and keeps what its three checks compare
    the trainer with (tools/reference_check.py:125-184), so the comparison can be repeated where
    the reference tree is absent."""
    import importlib.util

    spec_ = importlib.util.spec_from_file_location("reference_check", os.path.join(tools_dir, "reference_check.py"))
    rc = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(rc)
    fix = {}
    for name in SHAPES:
        path = os.path.join(out_dir, f"export_{name}.safetensors")
        export(name, path)
        t, cfg = rc.read_safetensors(path)
        ref = rc.Reference(t, cfg)
        fix[f"{name}.loss"] = np.float64(ref.loss())
        def fd(move, eps):
            move(+eps)
            lp = ref.loss()
            move(-2 * eps)
            lm = ref.loss()
            move(+eps)
            return (lp - lm) / (2 * eps)

        for d_i in range(4):  # directions over every adapter weight at once, eps 1e-4
            dirs = directions(d_i, [(n, A.shape, B.shape) for n, (A, B) in ref.lora.items()])
            norm = 1.0  # directions() returns a unit vector

            def move(s):
                for n, (A, B) in ref.lora.items():
                    A += s * dirs[n][0] / norm
                    B += s * dirs[n][1] / norm

            fix[f"{name}.dir{d_i}.fd"] = np.float64(fd(move, 1e-4))
        names = list(ref.lora)
        rng = np.random.default_rng(7)
        coords = []
        for c in range(42):  # single entries, eps 1e-3, spread over modules, A and B in turn
            n = names[(c * 5) % len(names)]
            j = c % 2
            P = ref.lora[n][j]
            idx = tuple(int(rng.integers(0, s)) for s in P.shape)

            def move(s, P=P, idx=idx):
                P[idx] += s

            coords.append((names.index(n), j, idx[0], idx[1], fd(move, 1e-3)))
        fix[f"{name}.coords"] = np.array(coords, dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "reference_check_float64.npz"), **fix)


if __name__ == "__main__":
    args = sys.argv[1:]
    if args and args[0] == "--fixture":
        import tempfile

        with tempfile.TemporaryDirectory() as d:
            float64_fixture(args[1], d)
        print("wrote", os.path.join(HERE, "reference_check_float64.npz"))
    else:
        out_dir = args[0] if args else "."
        for nm in SHAPES:
            p = os.path.join(out_dir, f"export_{nm}.safetensors")
            export(nm, p)
            print("wrote", p)
