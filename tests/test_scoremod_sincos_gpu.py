"""GPU parity: B3 direct sigmoid, fractional exp2, paired sin/cos, RoPE tables and the fused RoPE rotation."""
import math

import numpy as np
import pytest

from util import assert_bits_equal, ref_call, to_bits, to_device, uniform_bits

pytestmark = pytest.mark.gpu


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


# ---- B3 ------------------------------------------------------------------------------------------

def test_b3_direct_config1_bit_exact(fpt, cuda, oracle):
    """Configuration 1: 2^24 bf16 scores U[-16,16) with 1% specials; bit-exact; error vs fp64 reported."""
    import torch
    bits = uniform_bits(1 << 24, -16.0, 16.0, "bf16")
    x = to_device(bits, "bf16", cuda)
    for log2_n in (12, 14):
        prob, grad = torch.empty_like(x), torch.empty_like(x)
        fpt.call("fpt_b3_sigmoid_direct", prob.data_ptr(), grad.data_ptr(), x.data_ptr(), x.numel(), 0, log2_n, stream())
        torch.cuda.synchronize()
        want_p, want_g = oracle.b3_direct(bits, log2_n, with_grad=True)
        assert_bits_equal(to_bits(prob), want_p, f"b3 prob log2n={log2_n}", bits)
        assert_bits_equal(to_bits(grad), want_g, f"b3 grad log2n={log2_n}", bits)
        only = torch.empty_like(x)
        fpt.call("fpt_b3_sigmoid_direct", only.data_ptr(), None, x.data_ptr(), x.numel(), 0, log2_n, stream())
        torch.cuda.synchronize()
        assert torch.equal(only.view(torch.int16), prob.view(torch.int16))
    xf = oracle.bf16_bits_to_f32(bits).astype(np.float64)
    finite = np.isfinite(xf) & (np.abs(xf) <= 6)
    err = np.abs(oracle.bf16_bits_to_f32(oracle.b3_direct(bits, 12)).astype(np.float64)[finite]
                 - 1 / (1 + np.exp(-(xf[finite] - math.log(4096)))))
    assert err.max() < 0.04  # the deployed fit's own worst case is 0.0328 at x = 6


def test_b3_all_patterns_and_f32_scores(fpt, cuda, oracle):
    import torch
    allbits = np.arange(65536, dtype=np.uint16)
    x = to_device(allbits, "bf16", cuda)
    out = torch.empty_like(x)
    fpt.call("fpt_b3_sigmoid_direct", out.data_ptr(), None, x.data_ptr(), x.numel(), 0, 12, stream())
    torch.cuda.synchronize()
    assert_bits_equal(to_bits(out), oracle.b3_direct(allbits, 12), "b3 every pattern", allbits)
    rng = np.random.default_rng(7)
    sf = (rng.standard_normal(100001) * 3).astype(np.float32)
    sf[:4] = [np.nan, np.inf, -np.inf, -0.0]
    s = torch.from_numpy(sf).to(cuda)
    prob = torch.empty(sf.size, dtype=torch.bfloat16, device=cuda)
    grad = torch.empty_like(prob)
    fpt.call("fpt_b3_sigmoid_direct", prob.data_ptr(), grad.data_ptr(), s.data_ptr(), s.numel(), 1, 12, stream())
    torch.cuda.synchronize()
    want_p, want_g = oracle.b3_direct(sf, 12, with_grad=True)
    assert_bits_equal(to_bits(prob), want_p, "b3 from f32")
    assert_bits_equal(to_bits(grad), want_g, "b3 grad from f32")


@pytest.mark.parametrize("log2_n", [12, 14])
def test_b3_evaluation_order_of_the_attention_kernels_all_patterns(fpt, cuda, oracle, log2_n):
    """The attention kernels run the cubic in another instruction order (both rows, one select afterwards, no lower
    clamp, floor inside the last multiply-add).  Every bf16 pattern: probabilities equal the oracle bit for bit; the
    coupled gradient too, except at -inf, where the unclamped derivative factor is +inf and 0 * inf gives NaN
    (the kernels never meet that lane: they convert fp32 scores with saturation, checked below)."""
    import torch
    allbits = np.arange(65536, dtype=np.uint16)
    x = to_device(allbits, "bf16", cuda)
    want_p, want_g = oracle.b3_direct(allbits, log2_n, with_grad=True)
    only = torch.empty_like(x)
    fpt.call("fpt_b3_sigmoid_direct_variant", only.data_ptr(), None, x.data_ptr(), x.numel(), 0, log2_n, 1, stream())
    prob, grad = torch.empty_like(x), torch.empty_like(x)
    fpt.call("fpt_b3_sigmoid_direct_variant", prob.data_ptr(), grad.data_ptr(), x.data_ptr(), x.numel(), 0, log2_n, 1, stream())
    torch.cuda.synchronize()
    assert_bits_equal(to_bits(only), want_p, "b3 late select, value only", allbits)
    assert_bits_equal(to_bits(prob), want_p, "b3 late select, value", allbits)
    got_g = to_bits(grad)
    differs = np.nonzero(got_g != want_g)[0]
    assert differs.tolist() == [0xFF80], [hex(i) for i in differs[:16]]
    assert want_g[0xFF80] == 0x0000 and (got_g[0xFF80] & 0x7FFF) > 0x7F80      # +0 in the deployed order, NaN here
    # fp32 scores, the form in which the attention backward meets the evaluator: specials included, no lane differs
    rng = np.random.default_rng(11)
    sf = (rng.standard_normal(200003) * 4).astype(np.float32)
    sf[:10] = [np.nan, np.inf, -np.inf, -0.0, 0.0, -3.4e38, 3.4e38, -6.0, 6.0, 1.25]
    s = torch.from_numpy(sf).to(cuda)
    prob = torch.empty(sf.size, dtype=torch.bfloat16, device=cuda)
    grad = torch.empty_like(prob)
    fpt.call("fpt_b3_sigmoid_direct_variant", prob.data_ptr(), grad.data_ptr(), s.data_ptr(), s.numel(), 1, log2_n, 1, stream())
    torch.cuda.synchronize()
    want_p, want_g = oracle.b3_direct(sf, log2_n, with_grad=True)
    assert_bits_equal(to_bits(prob), want_p, "b3 late select from f32")
    assert_bits_equal(to_bits(grad), want_g, "b3 late select gradient from f32")


# ---- exp2 ----------------------------------------------------------------------------------------

def test_exp2_hinge_bit_exact_and_native_close(fpt, cuda, oracle):
    import torch
    rng = np.random.default_rng(1234)
    xb = rng.uniform(0, 1, (1 << 20) + 5).astype(np.float16).view(np.uint16)
    x = to_device(xb, "fp16", cuda)
    for variant, cset in ((1, 0), (2, 1)):
        for repeats in (1, 4, 16):
            out = torch.empty_like(x)
            fpt.call("fpt_exp2_fraction", out.data_ptr(), x.data_ptr(), x.numel(), variant, repeats, stream())
            torch.cuda.synchronize()
            assert_bits_equal(to_bits(out), oracle.exp2_hinge(xb, cset, repeats), f"exp2 set{cset} x{repeats}", xb)
    allbits = np.arange(65536, dtype=np.uint16)
    xa = to_device(allbits, "fp16", cuda)
    out = torch.empty_like(xa)
    fpt.call("fpt_exp2_fraction", out.data_ptr(), xa.data_ptr(), xa.numel(), 1, 1, stream())
    torch.cuda.synchronize()
    assert_bits_equal(to_bits(out), oracle.exp2_hinge(allbits, 0), "exp2 every pattern", allbits)
    out = torch.empty_like(x)
    fpt.call("fpt_exp2_fraction", out.data_ptr(), x.data_ptr(), x.numel(), 0, 1, stream())
    torch.cuda.synchronize()
    rel = ((out.float() - torch.exp2(x.float())).abs() / torch.exp2(x.float())).max()
    assert float(rel) < 1e-3
    hinge = torch.empty_like(x)
    fpt.call("fpt_exp2_fraction", hinge.data_ptr(), x.data_ptr(), x.numel(), 1, 1, stream())
    torch.cuda.synchronize()
    rel = ((hinge.float() - torch.exp2(x.float())).abs() / torch.exp2(x.float())).max()
    assert float(rel) < 0.0115  # published max-rel 0.0109


@pytest.mark.parametrize("variant,bound", [(0, 8.9e-5), (1, 2.2e-2), (2, 2.7e-3), (3, 1.14e-2)])
def test_full_range_exp2_bit_exact_and_accurate(fpt, cuda, oracle, variant, bound):
    """The software exponentials that the attention kernel mixes with the special-function unit, as a flat kernel."""
    import torch
    rng = np.random.default_rng(77)
    edge = np.array([0.0, -0.0, 0.5, -0.5, 1.0, -1.0, 8.0, -126.0, -127.0, -1000.0, -np.inf, 127.0, 126.99999,
                     -124.5, 0.49999997, -0.49999997, 1.5, 2.5, -1.5, 1e-30, -1e-30, 2.9999998, -3.0000002], dtype=np.float32)
    for n in (1, 3, 4, 7, (1 << 20) + 3):
        xs = np.concatenate([edge, rng.uniform(-140, 127, n).astype(np.float32)])[:max(n, 1)] if n < 64 else \
            np.concatenate([edge, rng.uniform(-140, 127, n).astype(np.float32), rng.uniform(-30, 8, n).astype(np.float32)])
        x = torch.from_numpy(xs).to(cuda)
        out = torch.empty_like(x)
        fpt.call("fpt_exp2_full_f32", out.data_ptr(), x.data_ptr(), x.numel(), variant, stream())
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        want = oracle.exp2_full(xs, variant)
        bad = np.nonzero(got.view(np.uint32) != want.view(np.uint32))[0]
        assert bad.size == 0, (n, bad[:5], xs[bad[:5]], got[bad[:5]], want[bad[:5]])
        inside = xs >= -126
        rel = np.abs(got[inside].astype(np.float64) / np.exp2(xs[inside].astype(np.float64)) - 1)
        assert rel.max() < bound
        assert np.all(got[xs <= -127] < 1.2e-38) and np.all(got[xs <= -127] >= 0.0)   # +0 (0.989 * 2^-126 for the line of variant 1)
        if variant >= 2:        # endpoint-preserving fits: 2^n exactly at every integer, so rescaling steps compose
            ints = np.arange(-126, 128, dtype=np.float32)
            xi = torch.from_numpy(ints).to(cuda)
            oi = torch.empty(256, dtype=torch.float32, device=cuda)[:ints.size]
            fpt.call("fpt_exp2_full_f32", oi.data_ptr(), xi.data_ptr(), ints.size, variant, stream())
            torch.cuda.synchronize()
            assert np.array_equal(oi.cpu().numpy(), np.exp2(ints.astype(np.float64)).astype(np.float32))
    assert fpt.load().fpt_exp2_full_f32(None, None, 5, variant, None) != 0            # null pointers
    x = torch.zeros(9, dtype=torch.float32, device=cuda)
    assert fpt.load().fpt_exp2_full_f32(x.data_ptr() + 4, x.data_ptr(), 4, variant, None) != 0   # misaligned
    assert fpt.load().fpt_exp2_full_f32(x.data_ptr(), x.data_ptr(), 4, 7, None) != 0              # unknown variant


def test_exp2_error_metrics_equal_the_reference_benchmark(fpt, cuda):
    """The reference's stand-alone exp2 benchmark (compiled from its own source by `make -C oracle ref`) prints, for a
    fixed arithmetic input sequence, max-abs / max-rel / rms error of each evaluator against fp64 exp2 with nine
    significant digits.  The same three figures computed from this library's kernels on the same 2^21 inputs must
    print identically: a checksum over every output bit that reaches an error figure."""
    import re
    import subprocess
    from pathlib import Path

    import torch
    binary = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "benchmark_exp2_pwl2"
    if not binary.exists():
        pytest.skip("oracle/_ref/benchmark_exp2_pwl2 not built")
    printed = subprocess.run([str(binary)], capture_output=True, text=True, timeout=600, check=True).stdout
    theirs = {}
    for m in re.finditer(r"ERROR domain=(\S+) variant=(\S+) max_abs=(\S+) max_rel=(\S+) rmse=(\S+) samples=(\d+)", printed):
        theirs[(m.group(1), m.group(2))] = m.groups()[2:]
    pairs = 1 << 20

    def metrics(got, x):
        ref = np.exp2(x.astype(np.float64))
        err = np.abs(got.astype(np.float64) - ref)
        # the benchmark accumulates the squares in input order in a double; a pairwise sum may differ in the last
        # digits, so the root-mean-square figure is compared to 1e-7 relative and the two maxima exactly
        return "%.9g" % err.max(), "%.9g" % (err / np.abs(ref)).max(), float(np.sqrt(np.sum(err * err) / err.size)), str(err.size)

    i = np.arange(2 * pairs, dtype=np.int64)
    frac = ((i % 65521).astype(np.float32) / np.float32(65521.0)).astype(np.float16)
    full = np.float32(-16.0) * ((i % 1048573).astype(np.float32) / np.float32(1048573.0))
    x16 = torch.from_numpy(frac.view(np.int16)).to(cuda).view(torch.float16)
    x32 = torch.from_numpy(full).to(cuda)
    cases = []
    for variant, name in ((1, "pwl2_hinge"),):     # the polynomial evaluators; the native rows are hardware approximations
        out = torch.empty_like(x16)
        fpt.call("fpt_exp2_fraction", out.data_ptr(), x16.data_ptr(), x16.numel(), variant, 1, stream())
        cases.append((("fractional_h2", name), out.float().cpu().numpy(), frac.astype(np.float32)))
    for variant, name in ((0, "degree3"), (1, "pwl2_hinge")):
        out = torch.empty_like(x32)
        fpt.call("fpt_exp2_full_f32", out.data_ptr(), x32.data_ptr(), x32.numel(), variant, stream())
        cases.append((("full_f32", name), out.cpu().numpy(), full))
    torch.cuda.synchronize()
    for key, got, x in cases:
        assert key in theirs, (key, sorted(theirs))
        max_abs, max_rel, rms, count = metrics(got, x)
        assert (max_abs, max_rel, count) == (theirs[key][0], theirs[key][1], theirs[key][3]), (key, max_abs, max_rel, theirs[key])
        assert abs(rms / float(theirs[key][2]) - 1) < 1e-7, (key, rms, theirs[key][2])


# ---- sin/cos -------------------------------------------------------------------------------------

SINCOS_REF = {0: "launch_sincos_d3_d4_quarter_turn_fp16", 1: "launch_sincos_d3_d4_half_turn_fp16",
              2: "launch_sincos_d5_d4_half_turn_fp16", 3: "launch_sincos_d5_d6_half_turn_fp16",
              4: "launch_sincos_d7_d6_half_turn_fp16", 5: "launch_sincos_d3_d4_bf16",
              6: "launch_sincos_d3_d4_quarter_turn_bf16", 7: "launch_sincos_d3_d4_half_turn_bf16",
              8: "launch_sincos_d5_d6_half_turn_bf16", 9: "launch_sincos_d5_d4_half_turn_fp16_bf16"}


def angles(n, seed=1234, span=math.pi):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-span, span, n).astype(np.float32)
    a[:6] = [0.0, -0.0, math.pi, -math.pi, 1e-30, 3e-5][:min(6, n)]
    return a


@pytest.mark.parametrize("n", [(1 << 18) + 3, 64, 5])
def test_sincos_every_variant_bit_exact(fpt, cuda, oracle, n):
    import torch
    for span in (math.pi, 131072.0):
        a = angles(n, span=span)
        ad = torch.from_numpy(a).to(cuda)
        for variant in range(10):
            out = torch.empty(2, n, dtype=torch.int16, device=cuda)
            fpt.call("fpt_sincos", out.data_ptr(), ad.data_ptr(), n, variant, 0, stream())
            torch.cuda.synchronize()
            want_c, want_s = oracle.sincos_packed(variant, a)
            got = out.cpu().numpy().view(np.uint16)
            assert_bits_equal(got[0], want_c, f"cos variant {variant} span {span}")
            assert_bits_equal(got[1], want_s, f"sin variant {variant} span {span}")


def test_sincos_compute_probe_bit_exact(fpt, cuda, oracle):
    import torch
    n = 4096 + 3
    a = angles(n)
    ad = torch.from_numpy(a).to(cuda)
    for variant in (3, 8, 0):
        for iterations in (1, 16):
            out = torch.empty(2, n, dtype=torch.int16, device=cuda)
            fpt.call("fpt_sincos", out.data_ptr(), ad.data_ptr(), n, variant, iterations, stream())
            torch.cuda.synchronize()
            want_c, want_s = oracle.sincos_packed(variant, a, iterations)
            got = out.cpu().numpy().view(np.uint16)
            assert_bits_equal(got[0], want_c, f"cos probe v{variant} x{iterations}")
            assert_bits_equal(got[1], want_s, f"sin probe v{variant} x{iterations}")


def test_sincos_accuracy_and_native(fpt, cuda):
    """D5/D6 half-turn fp16 within 1.5e-3 of the true functions on [-pi, pi]; native control within 1e-3."""
    import torch
    a = torch.linspace(-math.pi, math.pi, 200001, device=cuda)
    for variant, tol in ((3, 1.5e-3), (10, 1e-3)):
        out = torch.empty(2, a.numel(), dtype=torch.float16, device=cuda)
        fpt.call("fpt_sincos", out.data_ptr(), a.data_ptr(), a.numel(), variant, 0, stream())
        torch.cuda.synchronize()
        assert float((out[0].double() - torch.cos(a.double())).abs().max()) < tol
        assert float((out[1].double() - torch.sin(a.double())).abs().max()) < tol


def test_sincos_reference_kernels_agree(fpt, cuda, ref_kernels):
    import torch
    n = 1 << 18
    for span in (math.pi, 8192.0):
        a = torch.from_numpy(angles(n, seed=5, span=span)).to(cuda)
        for variant, symbol in SINCOS_REF.items():
            ours = torch.empty(2, n, dtype=torch.int16, device=cuda)
            ref = torch.empty_like(ours)
            fpt.call("fpt_sincos", ours.data_ptr(), a.data_ptr(), n, variant, 0, stream())
            torch.cuda.synchronize()
            ref_call(ref_kernels, symbol, ref, a, n)
            torch.cuda.synchronize()
            assert_bits_equal(ours.cpu().numpy().view(np.uint16), ref.cpu().numpy().view(np.uint16), symbol)


# ---- RoPE ----------------------------------------------------------------------------------------

def increments(head_dim, theta=500000.0):
    freqs = theta ** (-np.arange(0, head_dim, 2, dtype=np.float64) / head_dim)
    return np.round(freqs * (2.0 ** 32) / (2 * math.pi)).astype(np.int64).astype(np.uint32)


def test_rope_tables_bit_exact_and_accurate(fpt, cuda, oracle, ref_kernels):
    import torch
    seq, head_dim = 1031, 128
    inc = increments(head_dim)
    incd = torch.from_numpy(inc.view(np.int32)).to(cuda)
    for kind, symbol in ((0, "launch_rope_sincos_fixed_half_turn_d5_d6_fp16"), (1, "launch_rope_sincos_fixed_d3_d4_fp16")):
        table = torch.empty(2, seq, inc.size, dtype=torch.float16, device=cuda)
        fpt.call("fpt_rope_table", table.data_ptr(), incd.data_ptr(), seq, inc.size, kind, 0, stream())
        torch.cuda.synchronize()
        assert_bits_equal(to_bits(table), oracle.rope_table(kind, inc, seq), f"rope table kind {kind}")
        ref = torch.empty_like(table)
        ref_call(ref_kernels, symbol, ref, incd, seq, inc.size)
        torch.cuda.synchronize()
        assert_bits_equal(to_bits(table), to_bits(ref), symbol)
        pos = np.arange(seq, dtype=np.float64)[:, None]
        ang = pos * (inc.astype(np.float64)[None, :] * 2 * math.pi / 2.0 ** 32)
        tol = 2.5e-3 if kind == 0 else 4e-3
        assert np.abs(table[0].double().cpu().numpy() - np.cos(ang)).max() < tol
        assert np.abs(table[1].double().cpu().numpy() - np.sin(ang)).max() < tol


@pytest.mark.parametrize("shape", [(2, 67, 4, 2, 128), (1, 16, 3, 1, 64), (1, 9, 1, 1, 8), (2, 130, 8, 8, 96)])
def test_rope_apply_bit_exact(fpt, cuda, oracle, shape):
    import torch
    B, S, Hq, Hk, D = shape
    rng = np.random.default_rng(B * S)
    inc = increments(D)
    incd = torch.from_numpy(inc.view(np.int32)).to(cuda)
    for dtype, dt in (("fp16", 0), ("bf16", 1)):
        qf = rng.standard_normal((B, S, Hq, D)).astype(np.float32)
        kf = rng.standard_normal((B, S, Hk, D)).astype(np.float32)
        if dtype == "fp16":
            qb, kb = qf.astype(np.float16).view(np.uint16), kf.astype(np.float16).view(np.uint16)
        else:
            qb, kb = oracle.f32_to_bf16_bits(qf), oracle.f32_to_bf16_bits(kf)
        q, k = to_device(qb, dtype, cuda), to_device(kb, dtype, cuda)
        qo = torch.empty(B, Hq, S, D, dtype=q.dtype, device=cuda)
        ko = torch.empty(B, Hk, S, D, dtype=q.dtype, device=cuda)
        fpt.call("fpt_rope_apply", qo.data_ptr(), ko.data_ptr(), q.data_ptr(), k.data_ptr(), incd.data_ptr(),
                 B, S, Hq, Hk, D, 0, dt, stream())
        torch.cuda.synchronize()
        want_q, want_k = oracle.rope_apply(qb, kb, inc, io_bf16=(dtype == "bf16"))
        assert_bits_equal(to_bits(qo), want_q, f"rope q {dtype} {shape}")
        assert_bits_equal(to_bits(ko), want_k, f"rope k {dtype} {shape}")


def test_rope_apply_reference_kernel_and_cached_table_agree(fpt, cuda, ref_kernels):
    import torch
    B, S, Hq, Hk, D = 2, 257, 8, 2, 128
    inc = increments(D)
    incd = torch.from_numpy(inc.view(np.int32)).to(cuda)
    q = torch.randn(B, S, Hq, D, device=cuda).to(torch.float16)
    k = torch.randn(B, S, Hk, D, device=cuda).to(torch.float16)
    qo, ko = torch.empty(B, Hq, S, D, dtype=q.dtype, device=cuda), torch.empty(B, Hk, S, D, dtype=q.dtype, device=cuda)
    rq, rk = torch.empty_like(qo), torch.empty_like(ko)
    fpt.call("fpt_rope_apply", qo.data_ptr(), ko.data_ptr(), q.data_ptr(), k.data_ptr(), incd.data_ptr(),
             B, S, Hq, Hk, D, 0, 0, stream())
    torch.cuda.synchronize()
    ref_call(ref_kernels, "launch_rope_apply_fixed_half_turn_d5_d6_fp16", rq, rk, q, k, incd, B, S, Hq, Hk, D)
    torch.cuda.synchronize()
    assert torch.equal(qo.view(torch.int16), rq.view(torch.int16))
    assert torch.equal(ko.view(torch.int16), rk.view(torch.int16))
    # the same rotation from a cached polynomial table gives the same bits
    table = torch.empty(2, S, D // 2, dtype=torch.float16, device=cuda)
    fpt.call("fpt_rope_table", table.data_ptr(), incd.data_ptr(), S, D // 2, 0, 0, stream())
    cq, ck = torch.empty_like(qo), torch.empty_like(ko)
    fpt.call("fpt_rope_apply", cq.data_ptr(), ck.data_ptr(), q.data_ptr(), k.data_ptr(), table.data_ptr(),
             B, S, Hq, Hk, D, 3, 0, stream())
    torch.cuda.synchronize()
    assert torch.equal(cq.view(torch.int16), qo.view(torch.int16)) and torch.equal(ck.view(torch.int16), ko.view(torch.int16))
    # real rotation check against fp64 complex multiplication
    ang = torch.arange(S, device=cuda, dtype=torch.float64)[:, None] * torch.from_numpy(
        inc.astype(np.float64) * 2 * math.pi / 2.0 ** 32).to(cuda)[None, :]
    qc = torch.view_as_complex(q.double().view(B, S, Hq, D // 2, 2)) * torch.polar(torch.ones_like(ang), ang)[None, :, None, :]
    want = torch.view_as_real(qc).reshape(B, S, Hq, D).transpose(1, 2)
    assert float((qo.double() - want).abs().max()) < 2e-2
