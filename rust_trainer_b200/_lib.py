"""ctypes binding of librt_b200.so (the C ABI declared in include/rt_b200.h).

There is no CPU fallback: if the library has not been built, or cannot be loaded, importing
any entry point raises.  Build it with `python -m rust_trainer_b200.build`.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "librt_b200.so"

OK = 0
DT_F32, DT_BF16, DT_F16 = 0, 1, 2
STATUS_NAMES = {
    0: "RT_OK", 1: "RT_ERR_BAD_SHAPE", 2: "RT_ERR_UNSUPPORTED_TYPE", 3: "RT_ERR_CUDA", 4: "RT_ERR_NCCL",
    5: "RT_ERR_DEVICE_WAIT_TIMEOUT", 6: "RT_ERR_BAD_INDEX", 7: "RT_ERR_BAD_ARG", 8: "RT_ERR_TOO_LARGE", 9: "RT_ERR_NONFINITE",
}


class RtError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class ModelConfig(C.Structure):
    """struct rt_model_config of include/rt_b200.h."""

    _fields_ = [(n, C.c_int32) for n in ("vocab", "hidden", "ff", "n_layers", "n_heads", "n_kv_heads", "head_dim", "rot_dim")] + \
               [(n, C.c_float) for n in ("rope_theta", "rope_freq_scale", "rms_eps")] + \
               [(n, C.c_int32) for n in ("rope_neox", "qk_norm", "tie_embeddings", "head_rows")]


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library once; raises if it is missing (no fallback path exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is not built; run `python -m rust_trainer_b200.build`")
        _lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def _declare(L: C.CDLL) -> None:
    vp, sz, i32, f32p = C.c_void_p, C.c_size_t, C.c_int32, C.POINTER(C.c_float)
    sig = {
        "rt_ctx_create": (i32, [C.c_int, C.POINTER(vp)]),
        "rt_ctx_destroy": (None, [vp]),
        "rt_last_error": (C.c_char_p, [vp]),
        "rt_ctx_synchronize": (i32, [vp]),
        "rt_ctx_stream": (vp, [vp]),
        "rt_ctx_set_stream": (i32, [vp, vp]),
        "rt_frozen_forward_dev": (i32, [vp, vp, C.c_int, sz, vp, C.c_int, C.c_int]),
        "rt_frozen_backward_input_dev": (i32, [vp, vp, C.c_int, sz, vp, C.c_int, C.c_int]),
        "rt_frozen_backward_input_dev_noalloc": (i32, [vp, vp, C.c_int, sz, vp, C.c_int, C.c_int]),
        "rt_ggml_nbytes": (sz, [C.c_int, sz, sz]),
        "rt_frozen_create": (i32, [vp, C.c_int, sz, sz, vp, sz, C.POINTER(vp)]),
        "rt_frozen_destroy": (None, [vp]),
        "rt_frozen_out_dim": (sz, [vp]),
        "rt_frozen_in_dim": (sz, [vp]),
        "rt_frozen_nbytes": (sz, [vp]),
        "rt_frozen_forward": (i32, [vp, f32p, sz, f32p]),
        "rt_frozen_backward_input": (i32, [vp, f32p, sz, f32p]),
        "rt_frozen_row": (i32, [vp, sz, f32p]),
    }
    i32p = C.POINTER(C.c_int32)
    u64 = C.c_uint64
    sig.update({
        "rt_linear_create": (i32, [vp, vp, f32p, C.c_char_p, C.POINTER(vp)]),
        "rt_linear_destroy": (None, [vp]),
        "rt_linear_attach_lora": (i32, [vp, C.c_int, C.c_float, f32p, f32p]),
        "rt_linear_set_lora_enabled": (i32, [vp, C.c_int]),
        "rt_linear_forward_dev": (i32, [vp, vp, sz, vp, C.c_int, C.c_int]),
        "rt_linear_backward_dev": (i32, [vp, vp, vp, vp, sz, vp, C.c_int]),
        "rt_linear_forward": (i32, [vp, f32p, sz, f32p]),
        "rt_linear_backward": (i32, [vp, f32p, f32p, sz, f32p]),
        "rt_lora_read": (i32, [vp, f32p, f32p, f32p, f32p]),
        "rt_lora_write": (i32, [vp, f32p, f32p]),
        "rt_lora_zero_grad": (i32, [vp]),
        "rt_linear_name": (C.c_char_p, [vp]),
        "rt_linear_in_dim": (sz, [vp]),
        "rt_linear_out_dim": (sz, [vp]),
        "rt_linear_lora_rank": (C.c_int, [vp]),
        "rt_model_create": (i32, [vp, C.POINTER(ModelConfig), C.POINTER(vp)]),
        "rt_model_destroy": (None, [vp]),
        "rt_model_set_tensor": (i32, [vp, C.c_char_p, C.c_int, sz, sz, vp, sz]),
        "rt_model_finalize": (i32, [vp]),
        "rt_model_attach_lora": (i32, [vp, C.c_int, C.c_float, C.c_char_p, u64, C.POINTER(sz)]),
        "rt_model_num_lora": (sz, [vp]),
        "rt_model_lora_linear": (vp, [vp, sz]),
        "rt_model_set_lora_enabled": (i32, [vp, C.c_int]),
        "rt_model_zero_grad": (i32, [vp]),
        "rt_model_forward_backward": (i32, [vp, i32p, i32p, i32, i32p, i32p, f32p, i32, f32p, i32p]),
        "rt_model_score": (i32, [vp, i32p, i32p, i32, i32p, i32p, i32, f32p, i32p, f32p]),
        "rt_model_forward_backward_layout": (i32, [vp, i32p, i32p, i32, i32p, i32p, i32p, i32p, f32p, i32, f32p, i32p]),
        "rt_model_score_layout": (i32, [vp, i32p, i32p, i32, i32p, i32p, i32p, i32p, i32, f32p, i32p]),
        "rt_model_stage_batch": (i32, [vp, i32p, i32p, i32, i32p, i32p, f32p, i32]),
        "rt_model_run_staged": (i32, [vp, C.c_int]),
        "rt_model_read_results": (i32, [vp, f32p, i32, i32p]),
        "rt_ctx_launch_count": (u64, [vp]),
        "rt_ctx_selftest_wait_timeout": (i32, [vp, u64]),
        "rt_ctx_set_profiling": (i32, [vp, C.c_int]),
        "rt_ctx_profile_read": (i32, [vp, C.POINTER(u64), C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
        "rt_model_grad_buffer": (i32, [vp, C.POINTER(vp), C.POINTER(sz)]),
        "rt_model_set_checkpointing": (i32, [vp, i32]),
        "rt_model_checkpointing": (i32, [vp]),
        "rt_optim_step": (i32, [vp] + [C.c_float] * 6 + [f32p]),
        "rt_optim_state_read": (i32, [vp, C.POINTER(u64), f32p, f32p]),
        "rt_optim_state_write": (i32, [vp, u64, f32p, f32p]),
    })
    i8p, u8p = C.POINTER(C.c_int8), C.POINTER(C.c_uint8)
    ci, cf = C.c_int, C.c_float
    sig.update({
        "rt_frozen_create_q8_0": (i32, [vp, sz, sz, f32p, i8p, C.POINTER(vp)]),
        "rt_model_argmax_layout": (i32, [vp, i32p, i32p, i32, i32p, i32p, i32p, i32, i32p]),
        "rt_comm_unique_id": (i32, [u8p, sz]),
        "rt_comm_init_rank": (i32, [vp, ci, ci, u8p, sz]),
        "rt_comm_destroy": (i32, [vp]),
        "rt_comm_size": (ci, [vp]),
        "rt_comm_rank": (ci, [vp]),
        "rt_comm_allreduce_f32": (i32, [vp, vp, sz]),
        "rt_model_allreduce_grads": (i32, [vp]),
        "rt_op_rmsnorm": (i32, [vp, f32p, f32p, sz, sz, cf, f32p]),
        "rt_op_rmsnorm_backward": (i32, [vp, f32p, f32p, f32p, sz, sz, cf, f32p]),
        "rt_op_qk_norm_rope": (i32, [vp, f32p, f32p, f32p, i32p, sz, ci, ci, ci, ci, ci, cf, cf, f32p, ci, f32p, f32p, cf,
                                     f32p, f32p, f32p]),
        "rt_op_qk_norm_rope_backward": (i32, [vp, f32p, f32p, f32p, f32p, f32p, i32p, sz, ci, ci, ci, ci, ci, cf, cf, f32p, ci,
                                              f32p, f32p, cf, f32p, f32p, f32p]),
        "rt_op_attention": (i32, [vp, f32p, f32p, f32p, i32p, sz, ci, ci, ci, f32p, f32p]),
        "rt_op_attention_backward": (i32, [vp, f32p, f32p, f32p, f32p, i32p, sz, ci, ci, ci, f32p, f32p, f32p]),
        "rt_op_swiglu": (i32, [vp, f32p, f32p, sz, sz, f32p]),
        "rt_op_swiglu_backward": (i32, [vp, f32p, f32p, f32p, sz, sz, f32p, f32p]),
        "rt_op_cross_entropy": (i32, [vp, f32p, sz, sz, i32p, f32p, f32p, i32p, i32p, f32p]),
    })
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args


def declared_symbols() -> list[str]:
    """Names of every function include/rt_b200.h declares (parsed from the header)."""
    import re

    text = (_HERE.parent / "include" / "rt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", text)))
