"""CPU restatement of the reference's own vectorised arithmetic replays (test and benchmark infrastructure).

The reference has no CPU implementation of its packed kernels; what it does run on the CPU, besides PyTorch's native
functions, are the replays its coefficient fitters score candidates with.  They round the multiply and the add of every
Horner step separately, so they are NOT the single-rounding arithmetic of the kernels (that is what `oracle.py` models
exactly); they are restated here because they are the reference's CPU path for these functions and the benchmark
times them as such:

  * `horner_split_rounded_fp16`   numpy float16          reference: autonumerics_zero/evolution/fit_all_degrees.py:59-96
  * `horner_split_rounded_bf16`   torch bfloat16         reference: autonumerics_zero/evolution/fit_all_degrees_bf16.py:65-117
  * the way the fitter drives them (argument clamped to Lc, value of the odd part only): fit_all_degrees.py:121-127

`activation_replay_fp16` adds the steps that turn the odd part into the function on signed inputs (sign, + 1/2, the
SiLU form of the kernels) in float64, as the fitters' targets do (fit_all_degrees.py:31-48).  The paired sin/cos replay
of the reference, `polynomial_sincos` (src/sfu_repro/rope/polynomial_sincos.py:138-165), is part of the package's
Python surface (`sfu_repro.rope.polynomial_sincos`) and is timed from there.

Only tests and bench.py's CPU legs may import this module.
"""
from __future__ import annotations

import numpy as np

# (Lc, c1..cn) of the deployed fp16 programs the benchmark sweeps (reference: autonumerics_zero/spline_ops/
# spline_structs_odd.cuh:14-37 sigmoid D3, :154-178 tanh D4, :242-261 SiLU D3 = x * sigmoid-D3 form)
DEPLOYED_FP16 = {
    "sigmoid": (6.25, (0.28125, -0.0534362793, 0.0033779144)),
    "tanh": None,      # filled from the program table on first use (keeps one source of constants)
    "silu": (6.25, (0.28125, -0.0534362793, 0.0033779144)),
}


def horner_split_rounded_fp16(t_f64: np.ndarray, coeffs_fp16, is_odd: bool = True) -> np.ndarray:
    """Horner evaluation in numpy float16 with the product and the sum of every step rounded separately.

    `coeffs_fp16[i]` is the coefficient of t^i.  Odd: ((c_n t + c_{n-1}) t + ... + c_1) t with c_0 ignored; even:
    (...(c_n t + c_{n-1}) t + ...) t + c_0.  Returns float64."""
    t = np.asarray(t_f64).astype(np.float16)
    c = [np.float16(v) for v in coeffs_fp16]
    n = len(c) - 1
    acc = (t * c[n]).astype(np.float16)
    acc = (acc + c[n - 1]).astype(np.float16)
    for i in range(n - 2, 0 if is_odd else -1, -1):
        acc = (t * acc).astype(np.float16)
        acc = (acc + c[i]).astype(np.float16)
    if is_odd:
        acc = (t * acc).astype(np.float16)
    return acc.astype(np.float64)


def horner_split_rounded_bf16(t_f64: np.ndarray, coeffs_f64, is_odd: bool = True) -> np.ndarray:
    """The same replay on torch bfloat16 tensors (numpy has no bfloat16); coefficients are rounded to bf16 first."""
    import torch
    t = torch.from_numpy(np.array(t_f64, dtype=np.float64)).to(torch.bfloat16)
    c = [torch.tensor(float(v), dtype=torch.float64).to(torch.bfloat16) for v in coeffs_f64]
    n = len(c) - 1
    acc = (t * c[n]).to(torch.bfloat16)
    acc = (acc + c[n - 1]).to(torch.bfloat16)
    for i in range(n - 2, 0 if is_odd else -1, -1):
        acc = (t * acc).to(torch.bfloat16)
        acc = (acc + c[i]).to(torch.bfloat16)
    if is_odd:
        acc = (t * acc).to(torch.bfloat16)
    return acc.to(torch.float64).numpy()


def _tanh_constants():
    if DEPLOYED_FP16["tanh"] is None:
        from . import oracle
        row = oracle.program_table()[oracle.find_program("TANH_FWD_D4", oracle.FP16)]
        coeffs = oracle.f16_from_bits(np.array(row["coeffs"][:4], dtype=np.uint16)).astype(np.float64)
        clamp = float(oracle.f16_from_bits(np.array([row["clamp"]], dtype=np.uint16))[0])
        DEPLOYED_FP16["tanh"] = (clamp, tuple(float(v) for v in coeffs))
    return DEPLOYED_FP16["tanh"]


def activation_replay_fp16(name: str, x: np.ndarray) -> np.ndarray:
    """sigmoid / tanh / silu of fp16 inputs through the fitter's replay of the deployed fp16 program; float64 out."""
    clamp, coeffs = _tanh_constants() if name == "tanh" else DEPLOYED_FP16[name]
    xf = np.asarray(x).astype(np.float64)
    odd = horner_split_rounded_fp16(np.minimum(np.abs(xf), clamp), (0.0, *coeffs), is_odd=True)
    signed = np.copysign(odd, xf)
    if name == "tanh":
        return signed
    sig = signed + 0.5
    return sig if name == "sigmoid" else xf * sig
