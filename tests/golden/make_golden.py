#!/usr/bin/env python3
"""Generate the committed golden lane vectors (run once, here, by hand).

    python tests/golden/make_golden.py

Two independent sources pin the C oracle (and through it the CUDA kernels):

1. ``reference_pins``: known answers that the reference's own tests and paper
   state for this path (cited per entry), plus the table of effective 16-bit
   constants and input/output pairs that were worked out with exact rational
   arithmetic when the reference was surveyed.
2. ``fraction_model``: input/output pairs for every program in
   ``program_table.json`` computed by the exact-rational lane model below
   (``fractions.Fraction``; one rounding per fma/mul/add) -- a second
   restatement that shares no code with the C oracle.

Outputs: ``tests/golden/lane_vectors.json``.
"""
from __future__ import annotations

import json
import random
import sys
from fractions import Fraction
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1] / "oracle"))
from exact_float import BF16, FP16, bits_to_fraction, round_to_format  # noqa: E402

NAN = 0x7FFF


class Lane:
    """Exact model of one packed 16-bit lane (fp16 or bf16)."""

    def __init__(self, fmt):
        self.fmt = fmt
        self.inf = 0x7C00 if fmt == FP16 else 0x7F80
        self.half = 0x3800 if fmt == FP16 else 0x3F00
        self.one = 0x3C00 if fmt == FP16 else 0x3F80

    def dec(self, bits):
        return bits_to_fraction(bits, self.fmt)

    def is_nan(self, bits):
        return self.dec(bits) == "nan"

    def _enc(self, value: Fraction, zero_sign: int) -> int:
        if value == 0:
            return zero_sign << 15
        bits, _ = round_to_format(value, self.fmt)
        return bits

    def fma(self, a, b, c):
        da, db, dc = self.dec(a), self.dec(b), self.dec(c)
        if "nan" in (da, db, dc):
            return NAN
        sp = ((a ^ b) >> 15) & 1
        sc = (c >> 15) & 1
        a_inf, b_inf, c_inf = (isinstance(d, str) for d in (da, db, dc))
        if a_inf or b_inf:
            if (not a_inf and da == 0) or (not b_inf and db == 0):
                return NAN
            if c_inf and sc != sp:
                return NAN
            return (sp << 15) | self.inf
        if c_inf:
            return c
        prod = da * db
        total = prod + dc
        if total == 0:
            if prod == 0 and dc == 0:
                return (sp << 15) if sp == sc else 0
            return 0
        return self._enc(total, 0)

    def mul(self, a, b):
        da, db = self.dec(a), self.dec(b)
        if "nan" in (da, db):
            return NAN
        s = ((a ^ b) >> 15) & 1
        if isinstance(da, str) or isinstance(db, str):
            if (not isinstance(da, str) and da == 0) or (not isinstance(db, str) and db == 0):
                return NAN
            return (s << 15) | self.inf
        return self._enc(da * db, s)

    def add(self, a, b):
        da, db = self.dec(a), self.dec(b)
        if "nan" in (da, db):
            return NAN
        sa, sb = a >> 15, b >> 15
        if isinstance(da, str) or isinstance(db, str):
            if isinstance(da, str) and isinstance(db, str) and sa != sb:
                return NAN
            return a if isinstance(da, str) else b
        total = da + db
        if total == 0:
            return (sa << 15) if (da == 0 and db == 0 and sa == sb) else 0
        return self._enc(total, 0)

    def sub(self, a, b):
        return self.add(a, b ^ 0x8000)

    @staticmethod
    def _key(bits):
        return -(bits & 0x7FFF) - 1 if bits & 0x8000 else bits

    def min(self, a, b):
        na, nb = self.is_nan(a), self.is_nan(b)
        if na and nb:
            return NAN
        if na:
            return b
        if nb:
            return a
        return a if self._key(a) <= self._key(b) else b

    def max(self, a, b):
        na, nb = self.is_nan(a), self.is_nan(b)
        if na and nb:
            return NAN
        if na:
            return b
        if nb:
            return a
        return a if self._key(a) >= self._key(b) else b


def eval_program(row, x):
    L = Lane(FP16 if row["dtype"] == "fp16" else BF16)
    shape, d, c = row["shape"], row["degree"], row["coeffs"]
    if shape == "ALG_SIG":
        return L.mul(x, L.sub(L.one, x))
    if shape == "ALG_TANH":
        return L.sub(L.one, L.mul(x, x))
    sign, a = x & 0x8000, x & 0x7FFF
    t = L.min(a, row["clamp"])
    if shape == "EVEN":
        r = L.fma(t, c[d], c[d - 1])
        for k in range(d - 2, -1, -1):
            r = L.fma(t, r, c[k])
        return r
    h = L.fma(t, c[d - 1], c[d - 2])
    for k in range(d - 3, -1, -1):
        h = L.fma(t, h, c[k])
    h = L.mul(t, h)
    if shape == "ODD":
        return h ^ sign
    if shape == "ODD_SAT":
        return L.min(h, L.one) ^ sign
    if shape == "ODD_HALF":
        return L.add(L.half, h ^ sign)
    if shape == "XMUL_HALF":
        return L.mul(x, L.add(L.half, h ^ sign))
    if shape == "SWISH":
        return L.fma(a, h, L.mul(L.half, x))
    raise ValueError(shape)


B3_ROW0 = [0x3980, 0x3987, 0x3909, 0x37E8]
B3_ROW1 = [0xBB09, 0x3B8C, 0xBB11, 0x3A09]
B3_GRAD0 = [0x3F80, 0xBC10]
B3_GRAD1 = [0x3F81, 0xBB38]


def eval_b3(x, log2_n=12):
    L = Lane(BF16)
    dx = L.dec(x)
    row = (not L.is_nan(x)) and (dx == "inf" or (dx != "-inf" and dx >= Fraction(5, 4)))
    c = L.max(L.min(x, 0x40C0), 0xC0C0)
    k = [v - ((log2_n - 12) << 7) for v in (B3_ROW1 if row else B3_ROW0)]
    v = k[3]
    for coeff in (k[2], k[1], k[0]):
        v = L.fma(c, v, coeff)
    v = L.max(v, 0)
    g = B3_GRAD1 if row else B3_GRAD0
    grad = L.mul(v, L.fma(c, g[1], g[0]))
    return v, grad


def eval_exp2_hinge(x, consts):
    L = Lane(FP16)
    hinge = L.max(L.sub(x, 0x3800), 0)
    base = L.fma(x, consts[0], consts[1])
    return L.fma(hinge, consts[2], base)


def sample_inputs(fmt, rng, count):
    specials = [0x0000, 0x8000, 0x0001, 0x8001, 0x7FFF, 0xFFFF]
    if fmt == FP16:
        specials += [0x7C00, 0xFC00, 0x03FF, 0x83FF, 0x0400, 0x3C00, 0xBC00, 0x7BFF, 0xFBFF, 0x7E00, 0x7C01]
        lo, hi = -10.0, 10.0
    else:
        specials += [0x7F80, 0xFF80, 0x007F, 0x807F, 0x0080, 0x3F80, 0xBF80, 0x7F7F, 0xFF7F, 0x7FC0, 0x7F81]
        lo, hi = -10.0, 10.0
    out = list(specials)
    for _ in range(count):
        v = Fraction(rng.uniform(lo, hi))
        bits, _ = round_to_format(v, fmt)
        out.append(bits)
    for _ in range(count // 4):  # raw patterns: any exponent, subnormals, NaN payloads
        out.append(rng.getrandbits(16))
    return out


# Known answers stated by the reference (files inside the reference project).
REFERENCE_PINS = {
    # tests/test_audit_b3_deployed_fit.py:17-20
    "round_bf16": [[1.00390625, 1.0], [1.01171875, 1.015625]],
    # tests/test_audit_b3_deployed_fit.py:33-40 (rows before the 1/4096 scaling)
    "b3_rows": [[1.0, 1.0546875, 0.53515625, 0.11328125], [-8.5625, 17.5, -9.0625, 2.140625]],
    "b3_grad_factors": [[1.0, -0.0087890625], [1.0078125, -0.0028076171875]],
    # extras/paper/manuscript/main.tex:1046-1067 (bf16 immediates of the deployed PTX)
    "b3_ptx_split": 0x3FA0, "b3_ptx_clamp": [0x40C0, 0xC0C0],
    "b3_ptx_row0": B3_ROW0, "b3_ptx_row1": B3_ROW1,
    # extras/paper/manuscript/main.tex:1108-1111
    "b3_ptx_grad0": B3_GRAD0, "b3_ptx_grad1": B3_GRAD1,
    # tests/test_audit_b3_deployed_fit.py:53-79: f(0) = bf16(1/4096); f saturates beyond +-6
    "b3_lane": [[0x0000, 0x3980], [0x3F80, 0x3A2D], [0x3FA0, 0x3A54], [0x4040, 0x3BA1], [0x40C0, 0x3D69],
                [0x41A0, 0x3D69], [0xC040, 0x0000], [0xC0C0, 0x0000], [0xC1A0, 0x0000]],
    # autonumerics_zero/spline_ops/test_spline_ops.py:159-166: bf16 swish(x)*1 at [-100,-20,20,100] = [0,0,20,100] for D3..D6
    "bf16_swish_tails": {"in": [0xC2C8, 0xC1A0, 0x41A0, 0x42C8], "out_value": [0.0, 0.0, 20.0, 100.0]},
    # autonumerics_zero/cuda_benchmarks/benchmark_exp2_pwl2.cu:90-98 and extras/paper/manuscript/appendix_exp2.tex:72-76
    "exp2_sets": [[0x3A91, 0x3BEA, 0x357B], [0x3A62, 0x3C00, 0x3676]],
    # input/output pairs worked out with exact rational arithmetic during the survey of the reference
    "lane": {
        "SIGMOID_FWD_D3/fp16": [[0x0000, 0x3800], [0x3800, 0x3906], [0x3C00, 0x39DA], [0xBC00, 0x344D], [0x4200, 0x3BA2],
                                [0xC200, 0x29E0], [0x4640, 0x3BF7], [0x4800, 0x3BF7], [0xC800, 0x1C80]],
        "SWISH_FWD_D3/fp16": [[0x3800, 0x3506], [0x3C00, 0x39DA], [0xBC00, 0xB44D], [0x4200, 0x41BA], [0xC200, 0xB068],
                              [0x4800, 0x47F7], [0xC800, 0xA880]],
        "TANH_FWD_D4/fp16": [[0x3400, 0x340E], [0x3800, 0x3764], [0x3C00, 0x3A0C], [0xBC00, 0xBA0C], [0x4000, 0x3BC0],
                             [0x4180, 0x3BF3], [0x4800, 0x3BF3], [0xC800, 0xBBF3]],
        "TANH_FWD_D4/bf16": [[0x3CA4, 0x3CB1], [0x3E80, 0x3E81], [0x3F00, 0x3EEC], [0x3F80, 0x3F42], [0xBF80, 0xBF42],
                             [0x4000, 0x3F76], [0x4030, 0x3F80], [0x4120, 0x3F80]],
        "SIGMOID_FWD_D3/bf16": [[0x0000, 0x3F00], [0x3F00, 0x3F21], [0x3F80, 0x3F3B], [0xBF80, 0x3E8A], [0x4040, 0x3F75],
                                [0xC040, 0x3D30], [0x40C0, 0x3F80], [0x4180, 0x3F80], [0xC180, 0x0000]],
        "SWISH_FWD_D3/bf16": [[0x3F00, 0x3EA1], [0x3F80, 0x3F3B], [0xBF80, 0xBE8A], [0x3FC0, 0x3F9C], [0xBFC0, 0xBE90],
                              [0x4040, 0x4038], [0xC040, 0xBE04], [0x41A0, 0x41A0], [0xC1A0, 0x0000]],
    },
    "exp2_hinge_set0": [[0x0000, 0x3BEA], [0x3400, 0x3CC7], [0x3800, 0x3D99], [0x3A00, 0x3EC3], [0x3BFE, 0x3FEC]],
    "effective_constants": {
        "SIGMOID_FWD_D3/fp16": [0x4640, 0x3480, 0xAAD7, 0x1AEB],
        "TANH_FWD_D4/fp16": [0x4180, 0x3C6D, 0xB5FF, 0x241E, 0x2009],
        "SIGMOID_FWD_D3/bf16": [0x40C0, 0x3E90, 0xBD5A, 0x3B5E],
        "TANH_FWD_D4/bf16": [0x4030, 0x3F8B, 0xBEA5, 0xBCBD, 0x3C87],
    },
}


def main() -> None:
    rng = random.Random(20260101)
    table = json.loads((HERE / "program_table.json").read_text())
    model = {}
    for row in table:
        fmt = FP16 if row["dtype"] == "fp16" else BF16
        xs = sample_inputs(fmt, rng, 96)
        key = f'{row["name"]}/{row["dtype"]}/{row["source"]}'
        model[key] = {"in": "".join(f"{x:04x}" for x in xs),
                      "out": "".join(f"{eval_program(row, x):04x}" for x in xs)}
    xs = sample_inputs(BF16, rng, 400)
    b3 = {}
    for log2_n in (12, 14):
        pairs = [eval_b3(x, log2_n) for x in xs]
        b3[str(log2_n)] = {"in": "".join(f"{x:04x}" for x in xs),
                           "prob": "".join(f"{p:04x}" for p, _ in pairs),
                           "grad": "".join(f"{g:04x}" for _, g in pairs)}
    xs = [round_to_format(Fraction(rng.random()), FP16)[0] for _ in range(300)] + sample_inputs(FP16, rng, 40)
    exp2 = {}
    for idx, consts in enumerate(REFERENCE_PINS["exp2_sets"]):
        exp2[str(idx)] = {"in": "".join(f"{x:04x}" for x in xs),
                          "out": "".join(f"{eval_exp2_hinge(x, consts):04x}" for x in xs)}
    doc = {"reference_pins": REFERENCE_PINS, "fraction_model": model, "fraction_model_b3": b3,
           "fraction_model_exp2": exp2}
    (HERE / "lane_vectors.json").write_text(json.dumps(doc, indent=0) + "\n")
    print("programs:", len(model), "bytes:", (HERE / "lane_vectors.json").stat().st_size)


if __name__ == "__main__":
    main()
