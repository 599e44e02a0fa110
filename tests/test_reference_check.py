"""The CPU oracle against the reference's own float64 checker (tools/reference_check.py).

The reference verifies its trainer by exporting a smooth model, its loss and its analytic LoRA
gradients (examples/export_reference.rs) and re-deriving them with an independent NumPy float64
decoder.  Here the oracle sits in the trainer's seat (tests/golden/make_reference_export.py
writes the exporter's file from the oracle's numbers) and must pass the checker's own three
thresholds (tools/reference_check.py:125-184): loss rel < 1e-5, directional finite-difference
error / |g| < 1e-5, single entries rel < 1e-2.

Two forms: the unmodified checker run as a program (only where the reference tree is mounted),
and the same comparisons against its committed float64 outputs (everywhere).
"""
import importlib.util
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_reference_export", os.path.join(HERE, "golden", "make_reference_export.py"))
mre = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mre)

CHECKER = "/root/reference/tools/reference_check.py"
FIXTURE = np.load(os.path.join(HERE, "golden", "reference_check_float64.npz"))


@pytest.mark.parametrize("shape", list(mre.SHAPES))
@pytest.mark.skipif(not os.path.exists(CHECKER), reason="reference tree not mounted")
def test_oracle_passes_the_reference_checker(shape, tmp_path):
    path = tmp_path / f"export_{shape}.safetensors"
    mre.export(shape, path)
    r = subprocess.run([sys.executable, CHECKER, str(path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("PASS"), r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("shape", list(mre.SHAPES))
def test_oracle_matches_the_checkers_float64_numbers(shape):
    spec_, cfg, smooth, adapters, tokens = mre.smooth_case(shape)
    loss, grads = mre.oracle_run(cfg, smooth, adapters, tokens)
    ref_loss = float(FIXTURE[f"{shape}.loss"])
    assert abs(loss - ref_loss) / abs(ref_loss) < 1e-5
    g64 = [(ga.astype(np.float64), gb.astype(np.float64)) for ga, gb in grads]
    gnorm = np.sqrt(sum((g * g).sum() for pair in g64 for g in pair))
    names = [ad["name"] for ad in adapters]
    for d_i in range(4):
        dirs = mre.directions(d_i, [(n, g64[i][0].shape, g64[i][1].shape) for i, n in enumerate(names)])
        analytic = sum((dirs[n][0] * g64[i][0]).sum() + (dirs[n][1] * g64[i][1]).sum() for i, n in enumerate(names))
        assert abs(analytic - float(FIXTURE[f"{shape}.dir{d_i}.fd"])) / gnorm < 1e-5
    worst = 0.0
    scale = max(float(np.abs(g).max()) for pair in g64 for g in pair)
    for ni, j, r, c, fd in FIXTURE[f"{shape}.coords"]:
        analytic = g64[int(ni)][int(j)][int(r), int(c)]
        if abs(fd) < 1e-3 * scale:  # the checker only judges entries whose gradient is not negligible
            assert abs(analytic - fd) < 1e-5 * scale
            continue
        worst = max(worst, abs(analytic - fd) / abs(fd))
    assert worst < 1e-2


def test_int8_activation_mode_is_a_small_perturbation():
    """Mode (ii) of the oracle (activations rounded to 8 bits per block before every quantised
    forward matmul, src/rie.rs:77-80) against mode (i): informative, it bounds what that rounding
    can explain of a difference from the reference binary."""
    from oracle import oracle as O
    from rust_trainer_b200 import synth

    spec_ = synth.preset("tiny-qwen3", quant="Q8_0", seed=3, w_std=0.05)
    tensors = synth.build_tensors(spec_)
    ads = synth.lora_adapters(spec_, 4, 8.0, 2, b_std=0.02)
    toks = synth.token_batch(spec_, 1, 40, 5)[0]
    tp, tt = synth.answer_targets(toks, 20)
    w = np.full(tp.size, 1.0 / tp.size, np.float32)
    res = []
    for on in (False, True):
        O.set_act_int8(on)
        try:
            om = O.OracleModel(spec_.config(), tensors)
            om.attach_lora(ads)
            om.zero_grad()
            lp, _ = om.forward_backward(toks, tp, tt, w)
            g = np.concatenate([np.concatenate([e["ga"].ravel(), e["gb"].ravel()]) for e in om.lora])
            res.append((lp.copy(), g))
            om.close()
        finally:
            O.set_act_int8(False)
    (lp0, g0), (lp1, g1) = res
    assert not np.array_equal(lp0, lp1)  # the switch does something
    assert np.max(np.abs(lp1 - lp0) / np.abs(lp0)) < 2e-2
    assert np.linalg.norm(g1 - g0) / np.linalg.norm(g0) < 5e-2
