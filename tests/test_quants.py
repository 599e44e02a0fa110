"""Block-format decode: the oracle's C decoders and the package's NumPy codecs against the
committed golden vectors (decoded by the independent `gguf` package) and, when that package is
importable, against it directly.  Bit exact: integer/byte work."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from rust_trainer_b200 import quants as Q

GOLD = os.path.join(os.path.dirname(__file__), "golden")
FORMATS = [Q.F16, Q.BF16, Q.Q8_0, Q.Q4_0, Q.Q4_K, Q.Q6_K]


@pytest.mark.parametrize("t", FORMATS, ids=[Q.NAMES[t] for t in FORMATS])
def test_decode_matches_golden(t):
    g = np.load(os.path.join(GOLD, f"blocks_{Q.NAMES[t]}.npz"))
    packed, ref = g["packed"], g["decoded"]
    assert int(g["ggml_type"]) == t
    rows, cols = ref.shape
    assert packed.shape == (rows, Q.row_bytes(t, cols))
    assert np.array_equal(Q.dequantize(packed, t, cols), ref)
    assert np.array_equal(O.dequant_rows(t, packed, rows, cols), ref)


@pytest.mark.parametrize("t", FORMATS, ids=[Q.NAMES[t] for t in FORMATS])
def test_decode_matches_gguf_package(t):
    gguf = pytest.importorskip("gguf")
    from gguf import quants as gq

    gt = {Q.F16: gguf.GGMLQuantizationType.F16, Q.BF16: gguf.GGMLQuantizationType.BF16, Q.Q8_0: gguf.GGMLQuantizationType.Q8_0,
          Q.Q4_0: gguf.GGMLQuantizationType.Q4_0, Q.Q4_K: gguf.GGMLQuantizationType.Q4_K, Q.Q6_K: gguf.GGMLQuantizationType.Q6_K}[t]
    rng = np.random.default_rng(t)
    x = (rng.standard_normal((16, 1024)) * 0.02).astype(np.float32)
    packed = Q.quantize(x, t)
    src = packed.view(np.float16) if t == Q.F16 else packed
    ref = np.asarray(gq.dequantize(src, gt), dtype=np.float32).reshape(16, 1024)
    assert np.array_equal(O.dequant_rows(t, packed, 16, 1024), ref)
    if t in (Q.Q8_0, Q.Q4_0, Q.BF16):  # the package can also encode these: same bytes
        assert np.array_equal(np.asarray(gq.quantize(x, gt)).reshape(16, -1).view(np.uint8), packed)


@pytest.mark.parametrize("t,tol", [(Q.F16, 1e-3), (Q.BF16, 8e-3), (Q.Q8_0, 1e-2), (Q.Q4_0, 0.15), (Q.Q4_K, 0.12), (Q.Q6_K, 0.04)])
def test_roundtrip_error_is_bounded(t, tol):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((8, 768 if t not in (Q.Q4_K, Q.Q6_K) else 1024)) * 0.02).astype(np.float32)
    y = Q.dequantize(Q.quantize(x, t), t, x.shape[1])
    assert np.abs(y - x).max() <= tol * np.abs(x).max()


def test_bad_row_length_is_refused():
    with pytest.raises(ValueError):
        Q.quantize(np.zeros((2, 48), np.float32), Q.Q4_0)
    with pytest.raises(ValueError):
        Q.quantize(np.zeros((2, 896), np.float32), Q.Q4_K)


def test_f16_bf16_known_answers():
    # reference src/safetensors.rs:180-182
    assert Q.dequantize(np.array([[0x00, 0x3C]], np.uint8), Q.F16, 1)[0, 0] == 1.0
    assert Q.dequantize(np.array([[0x00, 0xC0]], np.uint8), Q.F16, 1)[0, 0] == -2.0
    assert Q.dequantize(np.array([[0x80, 0x3F]], np.uint8), Q.BF16, 1)[0, 0] == 1.0
