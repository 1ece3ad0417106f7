#!/usr/bin/env python3
"""Extract the polynomial program table from the reference headers.

Run in the authoring container only (it reads the reference checkout):

    python oracle/gen_program_table.py /path/to/reference

It parses every ``struct ..._ODD/_EVEN`` evaluator in
``autonumerics_zero/spline_ops/spline_structs_odd.cuh`` (FP16),
``spline_structs_odd_bf16.cuh`` (BF16) and ``spline_structs_sollya_bf16.cuh``
(BF16, Sollya coefficient source), classifies the arithmetic shape of the
body, converts every decimal literal the way the compiler does
(decimal -> fp32 -> 16-bit, round to nearest even) and writes

  * ``fast_polynomial_transcendentals_b200/csrc/fpt_program_table.inc``
    (X-macro rows consumed by the CUDA library and by the C oracle), and
  * ``tests/golden/program_table.json`` (the same rows plus the source
    line of every struct, used by the CPU tests as the pinned copy).

No reference source text is copied: only names, clamp limits and coefficient
values are taken, and they are re-encoded as 16-bit hexadecimal patterns.
"""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from exact_float import BF16, FP16, literal_to_16bit  # noqa: E402

REPO = Path(__file__).resolve().parents[1]
HEADERS = (
    ("autonumerics_zero/spline_ops/spline_structs_odd.cuh", "fp16", "current"),
    ("autonumerics_zero/spline_ops/spline_structs_odd_bf16.cuh", "bf16", "current"),
    ("autonumerics_zero/spline_ops/spline_structs_sollya_bf16.cuh", "bf16", "sollya"),
)

# Arithmetic shapes (t = min(|x|, Lc), h = t*(c1 + t*(c2 + ...)), s = sign(x)):
#   ODD_HALF  : 0.5 + s*h                 sigmoid fwd, swish bwd, gelu bwd
#   ODD       : s*h                       tanh fwd (FP16), erf fwd
#   ODD_SAT   : s*min(h, 1)               tanh fwd (BF16)
#   SWISH     : fma(|x|, h, 0.5*x)        swish fwd direct form
#   XMUL_HALF : x*(0.5 + s*h)             gelu fwd, composed swish fwd
#   EVEN      : c0 + t*(c1 + t*(...))     sigmoid/tanh bwd
#   ALG_SIG   : y*(1-y)                   algebraic sigmoid bwd from y
#   ALG_TANH  : 1 - y*y                   algebraic tanh bwd from y


def classify(body: str) -> str:
    flat = re.sub(r"\s+", " ", re.sub(r"//.*", "", body))
    if "__hsub2(one, __hmul2(y, y))" in flat:
        return "ALG_TANH"
    if "__hmul2(y, __hsub2(one, y))" in flat:
        return "ALG_SIG"
    if "::evaluate(val)" in flat:
        return "COMPOSED"
    if "c0 =" in flat:
        return "EVEN"
    if "__hfma2(abs_val, h," in flat:
        return "SWISH"
    if "__hmul2(val, phi)" in flat:
        return "XMUL_HALF"
    if "__hmin2(h," in flat:
        return "ODD_SAT"
    if "__hadd2(" in flat:
        return "ODD_HALF"
    return "ODD"


def parse_header(path: Path, dtype: str, source: str):
    fmt = FP16 if dtype == "fp16" else BF16
    text = path.read_text()
    rows = {}
    for match in re.finditer(r"struct (\w+) \{(.*?)\n\};", text, re.S):
        name, body = match.group(1), match.group(2)
        line = text.count("\n", 0, match.start()) + 1
        shape = classify(body)
        base = re.sub(r"(_SOLLYA)?(_BF16)?$", "", name)
        base = re.sub(r"_(ODD|EVEN)$", "", base)
        row = {"name": base, "dtype": dtype, "source": source, "shape": shape,
               "ref": f"{path.name}:{line}", "struct": name}
        if shape in ("ALG_SIG", "ALG_TANH"):
            row.update(degree=0, clamp=0, coeffs=[])
        elif shape == "COMPOSED":
            inner = re.search(r"(\w+)::evaluate\(val\)", body).group(1)
            row["inner"] = inner
        else:
            clamp = re.search(r"__hmin2\(abs_val, __float2\w+_rn\(([^)]+)\)\)", body).group(1)
            coeffs = dict(re.findall(r"\bc(\d) = __float2\w+_rn\(([^)]+)\)", body))
            order = sorted(coeffs, key=int)
            row.update(
                degree=int(order[-1]),
                clamp=literal_to_16bit(clamp, fmt),
                coeffs=[literal_to_16bit(coeffs[k], fmt) for k in order],
                clamp_literal=clamp,
                coeff_literals=[coeffs[k] for k in order],
            )
            m = re.search(r"_D(\d)_", name)
            assert m and int(m.group(1)) == row["degree"], name
        rows[name] = row
    for row in rows.values():  # resolve x*sigmoid(x) compositions
        if row["shape"] == "COMPOSED":
            inner = rows[row.pop("inner")]
            assert inner["shape"] == "ODD_HALF"
            row.update(shape="XMUL_HALF", degree=inner["degree"], clamp=inner["clamp"],
                       coeffs=list(inner["coeffs"]), clamp_literal=inner["clamp_literal"],
                       coeff_literals=list(inner["coeff_literals"]))
    return list(rows.values())


def main() -> None:
    import os
    reference = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FPT_REFERENCE_ROOT", REPO.parent / "reference"))
    table = []
    for rel, dtype, source in HEADERS:
        table.extend(parse_header(reference / rel, dtype, source))
    lines = [
        "// Generated by oracle/gen_program_table.py from the reference headers.",
        "// Row: FPT_PROGRAM(NAME, DTYPE, SOURCE, SHAPE, DEGREE, CLAMP, C0..C6)",
        "// 16-bit patterns are the literal -> fp32 -> fp16/bf16 (RNE) images of the",
        "// reference's decimal constants; unused coefficient slots are 0.",
        "// For ODD*/SWISH/XMUL_HALF shapes slot k holds c(k+1); for EVEN slot k holds c(k).",
    ]
    for row in table:
        coeffs = row["coeffs"] + [0] * (7 - len(row["coeffs"]))
        lines.append(
            "FPT_PROGRAM({name}, {dt}, {src}, {shape}, {deg}, 0x{clamp:04x}, {cs})".format(
                name=row["name"], dt=row["dtype"].upper(), src=row["source"].upper(),
                shape=row["shape"], deg=row["degree"], clamp=row["clamp"],
                cs=", ".join(f"0x{c:04x}" for c in coeffs)))
    out = REPO / "fast_polynomial_transcendentals_b200/csrc/fpt_program_table.inc"
    out.write_text("\n".join(lines) + "\n")
    (REPO / "tests/golden/program_table.json").write_text(json.dumps(table, indent=1) + "\n")
    print(f"{len(table)} programs -> {out}")


if __name__ == "__main__":
    main()
