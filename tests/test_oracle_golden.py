"""CPU: the C oracle against the committed golden vectors and the reference's own pins."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).parent / "golden"
DT = {"fp16": 0, "bf16": 1}
SRC = {"current": 0, "sollya": 1}


def unhex(s):
    return np.array([int(s[i:i + 4], 16) for i in range(0, len(s), 4)], dtype=np.uint16)


@pytest.fixture(scope="module")
def vectors():
    return json.loads((GOLDEN / "lane_vectors.json").read_text())


def test_program_table_matches_fixture(oracle):
    """The table compiled into the oracle equals the rows extracted from the reference headers."""
    fixture = json.loads((GOLDEN / "program_table.json").read_text())
    table = oracle.program_table()
    assert len(table) == len(fixture) == 108
    for got, want in zip(table, fixture):
        assert got["name"] == want["name"]
        assert got["dtype"] == DT[want["dtype"]] and got["source"] == SRC[want["source"]]
        assert got["shape"] == want["shape"] and got["degree"] == want["degree"]
        assert got["clamp"] == want["clamp"]
        assert got["coeffs"][:len(want["coeffs"])] == want["coeffs"]


def test_effective_constants_pinned(oracle, vectors):
    by_key = {(r["name"], r["dtype"], r["source"]): r for r in oracle.program_table()}
    for key, consts in vectors["reference_pins"]["effective_constants"].items():
        name, dt = key.split("/")
        row = by_key[(name, DT[dt], 0)]
        assert [row["clamp"]] + row["coeffs"][:len(consts) - 1] == consts, key


def test_exact_rational_model_agrees_for_every_program(oracle, vectors):
    total = 0
    for key, v in vectors["fraction_model"].items():
        name, dt, src = key.split("/")
        prog = oracle.find_program(name, DT[dt], SRC[src])
        x, want = unhex(v["in"]), unhex(v["out"])
        got = oracle.unary(prog, x)
        assert np.array_equal(got, want), key
        total += x.size
    assert total > 10000


def test_reference_lane_pins(oracle, vectors):
    for key, pairs in vectors["reference_pins"]["lane"].items():
        name, dt = key.split("/")
        prog = oracle.find_program(name, DT[dt], 0)
        for x, y in pairs:
            assert oracle.eval_lane(prog, x) == y, (key, hex(x))


def test_bf16_swish_tails_are_exact(oracle, vectors):
    """swish(x)*1 at [-100,-20,20,100] is [0,0,20,100] for D3..D6 (reference test_spline_ops.py:159-166)."""
    pin = vectors["reference_pins"]["bf16_swish_tails"]
    one = np.full(4, 0x3F80, dtype=np.uint16)
    for degree in (3, 4, 5, 6):
        prog = oracle.find_program(f"SWISH_FWD_D{degree}", 1, 0)
        out = oracle.swiglu(prog, np.array(pin["in"], dtype=np.uint16), one)
        assert oracle.bf16_bits_to_f32(out).tolist() == pin["out_value"], degree


def test_b3_direct_pins_and_model(oracle, vectors):
    pins = vectors["reference_pins"]
    for x, y in pins["b3_lane"]:
        assert oracle.b3_direct(np.array([x], dtype=np.uint16))[0] == y
    # f(0) == bf16(1/4096); saturation beyond the clamp (reference tests/test_audit_b3_deployed_fit.py:53-79)
    f = lambda v: oracle.b3_direct(oracle.f32_to_bf16_bits(np.array([v], dtype=np.float32)))[0]
    assert f(0.0) == 0x3980 and f(-20.0) == f(-6.0) and f(20.0) == f(6.0)
    # derivative factor is exactly 1.0 at 0: grad == value
    p, g = oracle.b3_direct(np.array([0], dtype=np.uint16), with_grad=True)
    assert p[0] == g[0]
    for log2_n, v in vectors["fraction_model_b3"].items():
        p, g = oracle.b3_direct(unhex(v["in"]), int(log2_n), with_grad=True)
        assert np.array_equal(p, unhex(v["prob"])) and np.array_equal(g, unhex(v["grad"]))


def test_b3_rows_scale_to_the_ptx_immediates(vectors):
    """Manifest rows x 2^-12 rounded to bf16 are the immediates of the deployed PTX."""
    pins = vectors["reference_pins"]
    from oracle.oracle import f32_to_bf16_bits
    for row, imm in ((pins["b3_rows"][0], pins["b3_ptx_row0"]), (pins["b3_rows"][1], pins["b3_ptx_row1"])):
        got = f32_to_bf16_bits(np.array(row, dtype=np.float32) / 4096.0)
        assert got.tolist() == imm
    for row, imm in ((pins["b3_grad_factors"][0], pins["b3_ptx_grad0"]), (pins["b3_grad_factors"][1], pins["b3_ptx_grad1"])):
        assert f32_to_bf16_bits(np.array(row, dtype=np.float32)).tolist() == imm
    for value, rounded in pins["round_bf16"]:
        got = f32_to_bf16_bits(np.array([value], dtype=np.float32))
        assert (got.astype(np.uint32) << 16).view(np.float32)[0] == rounded


def test_exp2_hinge_pins_and_model(oracle, vectors):
    for x, y in vectors["reference_pins"]["exp2_hinge_set0"]:
        assert oracle.exp2_hinge(np.array([x], dtype=np.uint16), 0)[0] == y
    for s, v in vectors["fraction_model_exp2"].items():
        assert np.array_equal(oracle.exp2_hinge(unhex(v["in"]), int(s)), unhex(v["out"]))
    # endpoint-preserving set: p(0) = 1 and p(1) = 2 exactly
    out = oracle.exp2_hinge(np.array([0x0000, 0x3C00], dtype=np.uint16), 1)
    assert out.tolist() == [0x3C00, 0x4000]


def test_full_range_exp2_restatements(oracle):
    """Floor reduction + cubic / two-piece line (the reference's FullDegree3 / FullPwl2Hinge sequences)."""
    xs = np.concatenate([np.linspace(-126, 127, 2_000_001), np.arange(-126, 128) + 0.5, np.arange(-126, 128) - 1e-6])
    xs = xs.astype(np.float32)
    xs = xs[(xs >= -126) & (xs <= 127)]
    truth = np.exp2(xs.astype(np.float64))
    d3 = oracle.exp2_full(xs, oracle.EXP2_FULL_D3).astype(np.float64)
    pwl = oracle.exp2_full(xs, oracle.EXP2_FULL_PWL2).astype(np.float64)
    assert np.abs(d3 / truth - 1).max() < 8.9e-5          # published for this cubic: 8.8e-5
    assert np.abs(pwl / truth - 1).max() < 2.2e-2
    ints = np.arange(-126, 128, dtype=np.float32)
    assert np.array_equal(oracle.exp2_full(ints, 0), np.exp2(ints.astype(np.float64)).astype(np.float32))   # f = 0: p = 1
    # below -127 the clamp holds, and the exponent field reaches zero there: the result is +0
    low = oracle.exp2_full(np.array([-127.0, -127.5, -1e6, -np.inf, np.nan], dtype=np.float32), 0)
    assert np.all(low == 0.0)
    low = oracle.exp2_full(np.array([-126.0, -127.5, -1e6, -np.inf, np.nan], dtype=np.float32), 1)
    assert np.all(low.view(np.uint32) == 0x007D4D54)     # the line clamps one exponent higher: p's mantissa, exponent field 0
    # subnormal inputs are zero (flush-to-zero on every step); the smallest normal negative rounds down to n = -1, f = 1
    tiny = oracle.exp2_full(np.array([-1e-40, 1e-40, -1e-30], dtype=np.float32), 0)
    assert tiny[0] == 1.0 and tiny[1] == 1.0 and 0.9999 < tiny[2] < 1.0
    # the fraction never leaves [0, 1): just below an integer the round-down add takes the lower integer
    x = np.nextafter(np.float32(3.0), np.float32(0.0))
    assert 7.99 < float(oracle.exp2_full(np.array([x], dtype=np.float32), 0)[0]) < 8.0


def test_endpoint_preserving_exp2_fits_reproduce_the_published_errors(oracle):
    """The two routed backends the reference retains: their maximum relative errors as published (quadratic 2.679e-3,
    packed fp16 two-piece line 1.132e-2 after coefficient rounding; reference: extras/paper/manuscript/
    appendix_exp2.tex:60-62 and :74-77), exact powers of two at every integer, +0 at and below the clamp."""
    xs = np.linspace(-20, 10, 2_000_001).astype(np.float32)
    truth = np.exp2(xs.astype(np.float64))
    for variant, published in ((oracle.EXP2_FULL_D2_SAFE, 2.679e-3), (oracle.EXP2_FULL_PWL2_SAFE_F16, 1.132e-2)):
        worst = np.abs(oracle.exp2_full(xs, variant).astype(np.float64) / truth - 1).max()
        assert abs(worst / published - 1) < 2e-3, (variant, worst)
        ints = np.arange(-126, 128, dtype=np.float32)
        assert np.array_equal(oracle.exp2_full(ints, variant), np.exp2(ints.astype(np.float64)).astype(np.float32))
        low = oracle.exp2_full(np.array([-127.0, -127.5, -1e6, -np.inf, np.nan], dtype=np.float32), variant)
        assert np.all(low.view(np.uint32) == 0)
    # a fraction that rounds to 1 in fp16 lands on the next power of two exactly (continuity across the integer)
    x = np.nextafter(np.float32(3.0), np.float32(0.0))
    assert float(oracle.exp2_full(np.array([x], dtype=np.float32), oracle.EXP2_FULL_PWL2_SAFE_F16)[0]) == 8.0


def test_error_ceilings_against_true_functions(oracle):
    """Published error bounds of the primary programs (struct comments / reference GPU checks)."""
    x = np.linspace(-15, 15, 30001).astype(np.float32)
    xh = x.astype(np.float16)
    sig = oracle.f16_from_bits(oracle.unary(oracle.find_program("SIGMOID_FWD_D3", 0), xh.view(np.uint16)))
    assert np.max(np.abs(sig.astype(np.float64) - 1 / (1 + np.exp(-xh.astype(np.float64))))) < 0.02
    th = oracle.f16_from_bits(oracle.unary(oracle.find_program("TANH_FWD_D4", 0), xh.view(np.uint16)))
    assert np.max(np.abs(th.astype(np.float64) - np.tanh(xh.astype(np.float64)))) < 0.0125
    xb = oracle.f32_to_bf16_bits(x)
    xbf = oracle.bf16_bits_to_f32(xb).astype(np.float64)
    sw = oracle.bf16_bits_to_f32(oracle.unary(oracle.find_program("SWISH_FWD_D3", 1), xb)).astype(np.float64)
    assert np.max(np.abs(sw - xbf / (1 + np.exp(-xbf)))) < 0.07
