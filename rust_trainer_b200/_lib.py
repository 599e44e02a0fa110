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
STATUS_NAMES = {
    0: "RT_OK", 1: "RT_ERR_BAD_SHAPE", 2: "RT_ERR_UNSUPPORTED_TYPE", 3: "RT_ERR_CUDA", 4: "RT_ERR_NCCL",
    5: "RT_ERR_DEVICE_WAIT_TIMEOUT", 6: "RT_ERR_BAD_INDEX", 7: "RT_ERR_BAD_ARG", 8: "RT_ERR_TOO_LARGE",
}


class RtError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


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
        "rt_frozen_forward_dev": (i32, [vp, vp, sz, vp, C.c_int, C.c_int]),
        "rt_frozen_backward_input_dev": (i32, [vp, vp, sz, vp, C.c_int, C.c_int]),
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
