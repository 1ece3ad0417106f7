"""CPU: the restated replays of the reference's CPU path (oracle/reference_replays.py, the package's
polynomial_sincos) against outputs of the reference's own functions (tests/golden/reference_replays.json, written by
tests/golden/make_replay_golden.py where the reference is present)."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "reference_replays.json").read_text())["cases"]


def arr(hex_bytes, dtype):
    return np.frombuffer(bytes.fromhex(hex_bytes), dtype=dtype)


@pytest.mark.parametrize("case", [c for c in GOLDEN if c["fn"] in ("fp16", "bf16")], ids=lambda c: f"{c['fn']}-{c['name']}-{c['is_odd']}")
def test_split_rounded_horner_equals_the_reference_function(case):
    from oracle import reference_replays as rr
    fn = rr.horner_split_rounded_fp16 if case["fn"] == "fp16" else rr.horner_split_rounded_bf16
    got = fn(arr(case["t"], np.float64), case["coeffs"], is_odd=case["is_odd"])
    assert np.array_equal(got.view(np.uint64), arr(case["out"], np.float64).view(np.uint64))


@pytest.mark.parametrize("case", [c for c in GOLDEN if c["fn"] == "sincos"], ids=lambda c: f"{c['name']}-{c['accurate']}")
def test_polynomial_sincos_equals_the_reference_function(case):
    import torch
    from fast_polynomial_transcendentals_b200.sfu_repro.rope import SOLLYA_D3_D4, UNIFORM_D7_D6, polynomial_sincos
    poly = {"sollya_d3_d4": SOLLYA_D3_D4, "uniform_d7_d6": UNIFORM_D7_D6}[case["name"]]
    cos, sin = polynomial_sincos(torch.from_numpy(arr(case["angles"], np.float32).copy()), polynomial=poly,
                                 accurate_reduction=case["accurate"])
    assert np.array_equal(cos.numpy().view(np.uint32), arr(case["cos"], np.float32).view(np.uint32))
    assert np.array_equal(sin.numpy().view(np.uint32), arr(case["sin"], np.float32).view(np.uint32))


def test_activation_replays_track_the_true_functions():
    """The fitter's replay of the deployed fp16 programs: within the programs' published error of the true functions."""
    from oracle import reference_replays as rr
    x = np.linspace(-12, 12, 20001).astype(np.float16)
    xf = x.astype(np.float64)
    assert np.abs(rr.activation_replay_fp16("sigmoid", x) - 1 / (1 + np.exp(-xf))).max() < 0.02
    assert np.abs(rr.activation_replay_fp16("tanh", x) - np.tanh(xf)).max() < 0.0135
    assert np.abs(rr.activation_replay_fp16("silu", x) - xf / (1 + np.exp(-xf))).max() < 0.08
