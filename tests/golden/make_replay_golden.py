"""Generates tests/golden/reference_replays.json by IMPORTING the reference's own replay functions.

    python tests/golden/make_replay_golden.py /path/to/reference

Runs where a checkout of the reference is present; the fixture it writes travels with the repository.  Inputs are
seeded; outputs are what `eval_horner_fp16_vec` / `eval_horner_bf16_vec` (reference: autonumerics_zero/evolution/
fit_all_degrees.py:59-96, fit_all_degrees_bf16.py:65-117) and `polynomial_sincos` (src/sfu_repro/rope/
polynomial_sincos.py:138-165) return for them, stored as hex of the float64 / float32 bytes.
"""
import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]


def main():
    reference = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FPT_REFERENCE_ROOT", ROOT.parent / "reference"))
    sys.path.insert(0, str(reference / "autonumerics_zero" / "evolution"))
    sys.path.insert(0, str(reference / "src"))
    import torch
    from fit_all_degrees import eval_horner_fp16_vec
    from fit_all_degrees_bf16 import eval_horner_bf16_vec
    from sfu_repro.rope.polynomial_sincos import SOLLYA_D3_D4, UNIFORM_D7_D6, polynomial_sincos

    rng = np.random.default_rng(20260902)
    cases = []
    coefficient_sets = {
        "sigmoid_d3": [0.0, 0.28125, -0.0534362793, 0.0033779144],
        "tanh_like_d4": [0.0, 1.0859375, -0.43505859375, 0.0755615234375, -0.004657745361328125],
        "even_d4": [0.25, 0.001, -0.02, 0.003, -0.0001],
        "d6": [0.0, 0.3, -0.05, 0.004, -0.0002, 1e-5, -1e-7],
    }
    for name, coeffs in coefficient_sets.items():
        for is_odd in (True, False):
            t = np.concatenate([rng.uniform(0, 8, 120), [0.0, 6.25, 1e-4, 6e-5, 8.0]])
            fp16_coeffs = [float(np.float16(c)) for c in coeffs]
            cases.append({"fn": "fp16", "name": name, "is_odd": is_odd, "coeffs": fp16_coeffs, "t": t.tobytes().hex(),
                          "out": np.asarray(eval_horner_fp16_vec(t, fp16_coeffs, is_odd=is_odd), dtype=np.float64).tobytes().hex()})
            cases.append({"fn": "bf16", "name": name, "is_odd": is_odd, "coeffs": coeffs, "t": t.tobytes().hex(),
                          "out": np.asarray(eval_horner_bf16_vec(t, coeffs, is_odd=is_odd), dtype=np.float64).tobytes().hex()})
    angles = np.concatenate([rng.uniform(-40, 40, 150), [0.0, np.pi / 4, -np.pi / 2, 3 * np.pi]]).astype(np.float32)
    for label, poly in (("sollya_d3_d4", SOLLYA_D3_D4), ("uniform_d7_d6", UNIFORM_D7_D6)):
        for accurate in (True, False):
            cos, sin = polynomial_sincos(torch.from_numpy(angles), polynomial=poly, accurate_reduction=accurate)
            cases.append({"fn": "sincos", "name": label, "accurate": accurate, "angles": angles.tobytes().hex(),
                          "cos": cos.numpy().astype(np.float32).tobytes().hex(), "sin": sin.numpy().astype(np.float32).tobytes().hex()})
    out = ROOT / "tests" / "golden" / "reference_replays.json"
    out.write_text(json.dumps({"generator": "tests/golden/make_replay_golden.py", "cases": cases}) + "\n")
    print(f"{len(cases)} cases -> {out}")


if __name__ == "__main__":
    main()
