"""Paired sine/cosine evaluators and RoPE helpers.  Importing this package patches nothing."""
from .polynomial_sincos import (SOLLYA_D3_D4, UNIFORM_D5_D4, UNIFORM_D7_D6, SincosPolynomial, evaluate_reduced_sincos,
                                polynomial_sincos, reduce_to_quarter_turn, rope_phase_increments)

__all__ = ["SOLLYA_D3_D4", "UNIFORM_D5_D4", "UNIFORM_D7_D6", "SincosPolynomial", "evaluate_reduced_sincos",
           "polynomial_sincos", "reduce_to_quarter_turn", "rope_phase_increments"]
