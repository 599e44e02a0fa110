"""Adapter files and training checkpoints (host side).

`write_gguf_adapter` / `read_gguf_adapter` restate the reference's engine-loadable LoRA file
(src/rie.rs:346-411; docs/ENGINE_LORA.md:19-37): keys `general.architecture`,
`general.type = "adapter"`, `adapter.type = "lora"`, `adapter.lora.alpha`, and per module
`<name>.weight.lora_a` (ggml ne [in, r]) and `<name>.weight.lora_b` (ne [r, out]) in F32, the
layout llama.cpp's `--lora` reads.  The GGUF container is written with the `gguf` package.

`save_checkpoint` / `load_checkpoint` write and read the trainer's own checkpoint file
(src/train.rs:389-455): one safetensors file with `<name>.A|B`, `.adam_m`, `.adam_v` per
trainable tensor and the loop state as the metadata entry `trainer_state`; a checkpoint taken
on other data or another configuration is refused; resuming continues bit for bit (every
kernel on the gradient path is deterministic).
"""
from __future__ import annotations

import json
import os

import numpy as np

GGUF_ADAPTER_FILE = "adapter.gguf"  # src/rie.rs:44


def write_gguf_adapter(model, path: str, arch: str, alpha: float | None = None) -> None:
    import gguf

    lins = model.lora_linears()
    if not lins:
        raise ValueError("no LoRA adapters")  # src/rie.rs:348
    tmp = str(path) + ".tmp"
    w = gguf.GGUFWriter(tmp, arch)
    w.add_string("general.type", "adapter")
    w.add_string("adapter.type", "lora")
    w.add_float32("adapter.lora.alpha", float(model.lora_alpha if alpha is None else alpha))
    for lin in lins:
        lo = lin.lora()
        w.add_tensor(f"{lin.name}.weight.lora_a", np.ascontiguousarray(lo["a"], dtype=np.float32))  # ne [in, r]
        w.add_tensor(f"{lin.name}.weight.lora_b", np.ascontiguousarray(lo["b"], dtype=np.float32))  # ne [r, out]
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    os.replace(tmp, path)  # atomic, like the reference's tmp + rename


def read_gguf_adapter(model, path: str, arch: str | None = None) -> int:
    """Replaces the model's adapters by the file's (src/rie.rs:369-411): every module the file
    names gets a fresh adapter of the file's rank with `adapter.lora.alpha` (the rank when the key
    is missing or 0), A and B from the file, enabled; modules the file does not name end up with
    no adapter.  Gradients and the optimiser state start from zero.  Returns the number of
    adapted modules.  Refuses a file that is not a LoRA adapter, is for another architecture,
    matches no module, or whose shapes do not fit.  One rank per file: the device keeps all
    adapters in one flat buffer attached with a single rank."""
    import gguf

    r = gguf.GGUFReader(path)

    def kv_str(key):
        f = r.fields.get(key)
        return None if f is None else bytes(f.parts[f.data[0]]).decode()

    if kv_str("adapter.type") != "lora":
        raise ValueError("not a LoRA adapter GGUF")
    file_arch = kv_str("general.architecture")
    if arch is not None and file_arch is not None and file_arch != arch:
        raise ValueError(f"adapter is for '{file_arch}', model is '{arch}'")
    f = r.fields.get("adapter.lora.alpha")
    alpha = 0.0 if f is None else float(f.parts[f.data[0]][0])
    tensors = {t.name: np.array(t.data, dtype=np.float32).reshape([int(d) for d in reversed(t.shape)]) for t in r.tensors}
    found = []
    for name, in_dim, out_dim in model.linear_shapes():
        a, b = tensors.get(f"{name}.weight.lora_a"), tensors.get(f"{name}.weight.lora_b")
        if a is None or b is None:
            continue
        if a.ndim != 2 or b.ndim != 2 or a.shape[1] != in_dim or b.shape[0] != out_dim or b.shape[1] != a.shape[0]:
            raise ValueError(f"{name}: adapter shape mismatch")
        found.append((name, a, b))
    if not found:
        raise ValueError("adapter matched no modules")
    ranks = {a.shape[0] for _, a, _ in found}
    if len(ranks) != 1:
        raise ValueError(f"adapter mixes ranks {sorted(ranks)}; one rank per file is supported")
    rank = ranks.pop()
    model.attach_lora(rank, alpha if alpha > 0.0 else float(rank), [n for n, _, _ in found])
    lins = {lin.name: lin for lin in model.lora_linears()}
    for name, a, b in found:
        lins[name].write_lora(a, b)
    return len(found)


def data_fingerprint(examples) -> int:
    """FNV-1a style hash over every example's token ids and answer_start (src/train.rs:158-176);
    `examples` yields (tokens, answer_start); for preference pairs feed chosen then rejected."""
    mask = (1 << 64) - 1
    h = 0xCBF29CE484222325
    for tokens, answer_start in examples:
        for t in np.asarray(tokens).reshape(-1).tolist():
            h = ((h ^ int(t)) * 0x100000001B3) & mask
        h = ((h ^ int(answer_start)) * 0x100000001B3) & mask
    return h


def _param_names(model) -> list:
    """optim.rs:32-34: `<linear name>.A`, `<linear name>.B` per adapted linear."""
    return [f"{lin.name}.{ab}" for lin in model.lora_linears() for ab in ("A", "B")]


def save_checkpoint(model, path: str, trainer_state: dict) -> None:
    """One safetensors file, as Trainer::save_checkpoint writes it (src/train.rs:389-406): per
    trainable tensor `<name>` (flat f32), `<name>.adam_m`, `<name>.adam_v`, and the metadata
    entry `trainer_state` holding the loop state as JSON (step, order, opt_t, losses,
    data_fingerprint, config_json, ...).  Written to a temporary file and renamed."""
    from safetensors.numpy import save_file

    t, m, v = model.optim_state()
    tensors = {}
    off = 0
    for lin in model.lora_linears():
        lo = lin.lora()
        for ab, key in (("A", "a"), ("B", "b")):
            w = np.ascontiguousarray(lo[key], dtype=np.float32).reshape(-1)
            n = f"{lin.name}.{ab}"
            tensors[n] = w
            tensors[n + ".adam_m"] = np.ascontiguousarray(m[off:off + w.size])
            tensors[n + ".adam_v"] = np.ascontiguousarray(v[off:off + w.size])
            off += w.size
    state = dict(trainer_state)
    state["opt_t"] = int(t)
    tmp = str(path) + ".tmp"
    save_file(tensors, tmp, metadata={"trainer_state": json.dumps(state)})
    os.replace(tmp, path)


def load_checkpoint(model, path: str, expect: dict | None = None) -> dict:
    """Trainer::load_checkpoint (src/train.rs:408-455).  `expect` is the state of the run that is
    resuming: the checkpoint is refused when its `data_fingerprint` or `config_json` differ
    ("training data changed since checkpoint" / "training config changed since checkpoint").
    Everything is read and checked before the model is touched."""
    from safetensors import safe_open

    with safe_open(path, framework="numpy") as f:
        md = f.metadata() or {}
        if "trainer_state" not in md:
            raise ValueError("no trainer_state")
        state = json.loads(md["trainer_state"])
        if expect is not None:
            if state.get("data_fingerprint") != expect.get("data_fingerprint"):
                raise ValueError("training data changed since checkpoint")
            if state.get("config_json") != expect.get("config_json"):
                raise ValueError("training config changed since checkpoint")
        lins = model.lora_linears()
        ws, ms, vs = [], [], []
        for lin in lins:
            lo_r, k, n_out = lin.rank, lin.in_dim(), lin.out_dim()
            for ab, size in (("A", lo_r * k), ("B", n_out * lo_r)):
                n = f"{lin.name}.{ab}"
                w = f.get_tensor(n)
                if w.size != size:
                    raise ValueError(f"{n}: shape changed")
                ws.append(w)
                ms.append(f.get_tensor(n + ".adam_m").reshape(-1))
                vs.append(f.get_tensor(n + ".adam_v").reshape(-1))
    for i, lin in enumerate(lins):
        lin.write_lora(ws[2 * i].reshape(lin.rank, lin.in_dim()), ws[2 * i + 1].reshape(lin.out_dim(), lin.rank))
    model.set_optim_state(state["opt_t"], np.concatenate(ms), np.concatenate(vs))
    return state
