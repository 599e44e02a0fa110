"""Adapter files and training checkpoints (host side).

`write_gguf_adapter` / `read_gguf_adapter` restate the reference's engine-loadable LoRA file
(src/rie.rs:346-411; docs/ENGINE_LORA.md:19-37): keys `general.architecture`,
`general.type = "adapter"`, `adapter.type = "lora"`, `adapter.lora.alpha`, and per module
`<name>.weight.lora_a` (ggml ne [in, r]) and `<name>.weight.lora_b` (ne [r, out]) in F32, the
layout llama.cpp's `--lora` reads.  The GGUF container is written with the `gguf` package.

`save_checkpoint` / `load_checkpoint` keep what src/train.rs:389-455 keeps: per adapter A and B,
the Adam moments, the optimiser step count and a JSON trainer state; resuming continues bit for
bit (every kernel on the gradient path is deterministic).
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
    """Loads A and B of every module the file names into the model's attached adapters; returns
    the number of adapted modules.  Refuses a file that is not a LoRA adapter, is for another
    architecture, or whose shapes do not fit (src/rie.rs:369-411)."""
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
    tensors = {t.name: np.array(t.data, dtype=np.float32).reshape([int(d) for d in reversed(t.shape)]) for t in r.tensors}
    n = 0
    for lin in model.lora_linears():
        a, b = tensors.get(f"{lin.name}.weight.lora_a"), tensors.get(f"{lin.name}.weight.lora_b")
        if a is None or b is None:
            continue
        if a.shape != (lin.rank, lin.in_dim()) or b.shape != (lin.out_dim(), lin.rank):
            raise ValueError(f"{lin.name}: adapter shape mismatch")
        lin.write_lora(a, b)
        n += 1
    if n == 0:
        raise ValueError("adapter matched no modules")
    return n


def save_checkpoint(model, path: str, trainer_state: dict) -> None:
    arrays = {}
    for lin in model.lora_linears():
        lo = lin.lora()
        arrays[f"{lin.name}.A"] = lo["a"]
        arrays[f"{lin.name}.B"] = lo["b"]
    t, m, v = model.optim_state()
    arrays["adam_m"], arrays["adam_v"] = m, v
    state = dict(trainer_state)
    state["opt_t"] = int(t)
    arrays["trainer_state"] = np.frombuffer(json.dumps(state).encode(), dtype=np.uint8)
    tmp = str(path) + ".tmp.npz"
    np.savez(tmp, **arrays)
    os.replace(tmp, path)


def load_checkpoint(model, path: str) -> dict:
    z = np.load(path)
    state = json.loads(bytes(z["trainer_state"]).decode())
    for lin in model.lora_linears():
        lin.write_lora(z[f"{lin.name}.A"], z[f"{lin.name}.B"])
    model.set_optim_state(state["opt_t"], z["adam_m"], z["adam_v"])
    return state
