"""The C-ABI library loads and exports every symbol include/rt_b200.h declares (no compute:
this runs without a GPU), and the entry points refuse work cleanly when no device exists."""
import ctypes as C
import re
from pathlib import Path

import pytest

from rust_trainer_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def test_library_is_built_in_tree():
    assert _lib.LIB_PATH.exists(), "run `python -m rust_trainer_b200.build` (or __graft_entry__.build())"
    assert ROOT in _lib.LIB_PATH.parents


def test_every_declared_symbol_is_exported():
    L = _lib.lib()
    declared = _lib.declared_symbols()
    assert len(declared) >= 45
    missing = [s for s in declared if not hasattr(L, s)]
    assert not missing, missing


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    text = (ROOT / "include" / "rt_b200.h").read_text()
    assert text.count("src/") >= 30
    for needle in ("src/frozen.rs:14-25", "src/linear.rs", "src/model.rs", "src/optim.rs", "src/rie.rs"):
        assert needle in text


def test_no_torch_types_in_the_abi():
    text = (ROOT / "include" / "rt_b200.h").read_text()
    assert "torch" not in text.lower() and "at::" not in text and "std::" not in text


def test_status_codes_match_python_table():
    text = (ROOT / "include" / "rt_b200.h").read_text()
    for code, name in _lib.STATUS_NAMES.items():
        assert re.search(rf"\b{name}\s*=\s*{code}\b", text), name


def test_ggml_nbytes_needs_no_device():
    L = _lib.lib()
    assert L.rt_ggml_nbytes(2, 4, 64) == 4 * 2 * 18      # Q4_0
    assert L.rt_ggml_nbytes(8, 4, 64) == 4 * 2 * 34      # Q8_0
    assert L.rt_ggml_nbytes(12, 3, 512) == 3 * 2 * 144   # Q4_K
    assert L.rt_ggml_nbytes(14, 3, 512) == 3 * 2 * 210   # Q6_K
    assert L.rt_ggml_nbytes(12, 3, 896) == 0             # not a multiple of the super-block
    assert L.rt_ggml_nbytes(3, 1, 32) == 0               # Q4_1: not supported


def test_context_creation_fails_loudly_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import rust_trainer_b200 as rt

    with pytest.raises(rt.RtError):
        rt.Context(0)
    assert _lib.lib().rt_last_error(None) == b"null context"


def test_product_never_imports_the_oracle():
    pkg = ROOT / "rust_trainer_b200"
    for f in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.h")) + list(pkg.rglob("*.cuh")):
        src = f.read_text()
        assert "import oracle" not in src and "from oracle" not in src and "liboracle" not in src, f
