"""Portable (any torch device) paired sin/cos by parity polynomials, used to build and to check RoPE tables.

Same interface and retained coefficient sets as the reference's evaluator (reference:
src/sfu_repro/rope/polynomial_sincos.py:13-78 coefficient sets, :90-126 range reduction, :129-165 evaluation):
sin(r) = r * P(r^2), cos(r) = Q(r^2) on a quarter-turn residual r in [-pi/4, pi/4], quadrant restored afterwards,
result returned as (cos, sin).  This is table-generation and checking code in fp32/fp64; the device kernels of this
package (`spline_ops.sincos_*`, `rope_*`) are the fast path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class SincosPolynomial:
    """Coefficients in r^2, lowest order first, valid on [-pi/4, pi/4]."""

    sin_coefficients: tuple[float, ...]
    cos_coefficients: tuple[float, ...]
    fit_name: str

    @property
    def sin_degree(self) -> int:
        return 2 * len(self.sin_coefficients) - 1

    @property
    def cos_degree(self) -> int:
        return 2 * len(self.cos_coefficients) - 2


# D3/D4: Sollya fpminimax with fp32 coefficients (bf16-grade rotation); D5/D4 and D7/D6: uniform least squares.
SOLLYA_D3_D4 = SincosPolynomial((0.9990314245223999, -0.16034401953220367),
                                (0.9999900460243225, -0.4997082054615021, 0.04039861634373665),
                                "sollya_fpminimax_d3_d4_f32")
UNIFORM_D5_D4 = SincosPolynomial((0.9999962449073792, -0.16661198437213898, 0.008137642405927181),
                                 (0.999993085861206, -0.499763548374176, 0.04051213711500168), "uniform_d5_d4_f32")
UNIFORM_D7_D6 = SincosPolynomial((1.0, -0.1666664183139801, 0.00833179522305727, -0.00019484198128338903),
                                 (1.0, -0.49999886751174927, 0.041656624525785446, -0.0013605882413685322),
                                 "uniform_d7_d6_f32")

_HALF_PI_HI_F32 = 1.570796251296997      # Cody-Waite split of pi/2 for the fp32 reducer
_HALF_PI_LO_F32 = 7.549789415861596e-08


def reduce_to_quarter_turn(angles: torch.Tensor, *, accurate: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """(residual fp32 in about [-pi/4, pi/4], quadrant in 0..3).

    accurate=True reduces in fp64 (for cached tables, where set-up accuracy matters); accurate=False is the two-term
    fp32 reduction a fused kernel would use, whose error grows with |angle|.
    """
    if not torch.is_floating_point(angles):
        raise TypeError("angles must be a floating-point tensor")
    work = angles.to(torch.float64 if accurate else torch.float32)
    turns = torch.round(work * (2.0 / math.pi))
    if accurate:
        residual = work - turns * (math.pi / 2.0)
    else:
        residual = (work - turns * _HALF_PI_HI_F32) - turns * _HALF_PI_LO_F32
    return residual.to(torch.float32), turns.to(torch.int64) & 3


def _poly(x: torch.Tensor, coefficients: tuple[float, ...]) -> torch.Tensor:
    acc = torch.full_like(x, coefficients[-1])
    for c in coefficients[-2::-1]:
        acc = acc * x + c
    return acc


def evaluate_reduced_sincos(reduced: torch.Tensor, polynomial: SincosPolynomial = UNIFORM_D7_D6):
    """(sin, cos) of an already reduced fp32 argument."""
    r = reduced.to(torch.float32)
    r2 = r * r
    return r * _poly(r2, polynomial.sin_coefficients), _poly(r2, polynomial.cos_coefficients)


def polynomial_sincos(angles: torch.Tensor, *, polynomial: SincosPolynomial = UNIFORM_D7_D6,
                      accurate_reduction: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """(cos, sin) from one shared range reduction; evaluation is fp32 whatever the angle dtype."""
    residual, quadrant = reduce_to_quarter_turn(angles, accurate=accurate_reduction)
    s, c = evaluate_reduced_sincos(residual, polynomial)
    odd = (quadrant & 1).bool()
    sin_mag, cos_mag = torch.where(odd, c, s), torch.where(odd, s, c)
    sin = torch.where((quadrant & 2).bool(), -sin_mag, sin_mag)
    cos = torch.where(((quadrant + 1) & 2).bool(), -cos_mag, cos_mag)
    return cos, sin


def rope_phase_increments(head_dim: int, theta: float = 500000.0, device=None) -> torch.Tensor:
    """int32 Q0.32 phase increments round(theta^(-2i/D) * 2^32 / 2pi), one per (even, odd) pair -- the parameter of
    the fixed-point RoPE kernels (reference: src/sfu_repro/rope/benchmark_cuda_fused_rope.py:237-241)."""
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim
    freqs = torch.pow(torch.tensor(theta, dtype=torch.float64), -exponents)
    inc = torch.round(freqs * (2.0 ** 32) / (2.0 * math.pi)).to(torch.int64)
    inc = torch.where(inc >= 2 ** 31, inc - 2 ** 32, inc).to(torch.int32)
    return inc if device is None else inc.to(device)
