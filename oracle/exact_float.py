"""Exact-rational floating point helpers (test infrastructure, not product code).

Everything here works on ``fractions.Fraction`` so that a value is rounded
exactly once, to nearest with ties to even, into a binary format described by
``(precision_bits, min_normal_exponent, max_exponent)``.  It is the slow,
obviously-correct model that the C oracle and the CUDA kernels are pinned to.

Formats (IEEE-754 style, subnormals kept, overflow to infinity):
  fp32: p=24, emin=-126, emax=127     fp16: p=11, emin=-14, emax=15
  bf16: p=8,  emin=-126, emax=127
"""
from __future__ import annotations

from fractions import Fraction

FP32 = (24, -126, 127)
FP16 = (11, -14, 15)
BF16 = (8, -126, 127)

_FIELDS = {FP32: (8, 23), FP16: (5, 10), BF16: (8, 7)}


def round_to_format(value: Fraction, fmt) -> tuple[int, Fraction]:
    """Round ``value`` to ``fmt``; return (bit pattern, rounded value).

    Infinity is reported as a bit pattern with the rounded value ``None``.
    The sign of an exact zero result is positive (callers that need IEEE
    signed-zero rules handle them before calling).
    """
    p, emin, emax = fmt
    ebits, mbits = _FIELDS[fmt]
    bias = (1 << (ebits - 1)) - 1
    sign = 1 if value < 0 else 0
    mag = -value if value < 0 else value
    if mag == 0:
        return 0, Fraction(0)
    # exponent e with 2^e <= mag < 2^(e+1)
    e = mag.numerator.bit_length() - mag.denominator.bit_length()
    if Fraction(2) ** e > mag:
        e -= 1
    if Fraction(2) ** (e + 1) <= mag:
        e += 1
    e = max(e, emin)
    quantum = Fraction(2) ** (e - (p - 1))
    scaled = mag / quantum
    q = scaled.numerator // scaled.denominator
    rem = scaled - q
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and (q & 1)):
        q += 1
    if q == (1 << p):  # carried into the next binade
        q >>= 1
        e += 1
    if e > emax:
        return (sign << (ebits + mbits)) | (((1 << ebits) - 1) << mbits), None
    rounded = q * Fraction(2) ** (e - (p - 1))
    if q < (1 << (p - 1)):  # subnormal or zero
        bits = q
    else:
        bits = ((e + bias) << mbits) | (q - (1 << (p - 1)))
    bits |= sign << (ebits + mbits)
    return bits, (-rounded if sign else rounded)


def bits_to_fraction(bits: int, fmt):
    """Decode a bit pattern; returns Fraction, or 'inf'/'-inf'/'nan'."""
    ebits, mbits = _FIELDS[fmt]
    bias = (1 << (ebits - 1)) - 1
    sign = (bits >> (ebits + mbits)) & 1
    e = (bits >> mbits) & ((1 << ebits) - 1)
    m = bits & ((1 << mbits) - 1)
    if e == (1 << ebits) - 1:
        if m:
            return "nan"
        return "-inf" if sign else "inf"
    if e == 0:
        v = Fraction(m) * Fraction(2) ** (1 - bias - mbits)
    else:
        v = (Fraction(m) + (1 << mbits)) * Fraction(2) ** (e - bias - mbits)
    return -v if sign else v


def literal_to_16bit(literal: str, fmt) -> int:
    """Decimal literal -> fp32 (as the compiler parses an ``f`` literal) -> 16-bit.

    This is the two-step rounding that ``__float2half2_rn(0.2810058594f)`` and
    ``__float2bfloat162_rn(...)`` perform on a source literal.
    """
    text = literal.strip().rstrip("fF")
    if "p" in text.lower():  # C hex-float literal such as 0x1p-15
        as_fraction = Fraction(float.fromhex(text))
    else:
        as_fraction = Fraction(text)
    _, f32 = round_to_format(as_fraction, FP32)
    bits, _ = round_to_format(f32, fmt)
    return bits
