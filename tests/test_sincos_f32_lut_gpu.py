"""GPU parity: the fp32 sin/cos family (eight polynomial variants + SFU control, with their repeated-evaluation
probes) and the table-look-up RoPE sin/cos, against the oracle and the reference's compiled kernels."""
import math

import numpy as np
import pytest

from util import assert_bits_equal, ref_call, to_bits

pytestmark = pytest.mark.gpu

VARIANTS = ("native", "d3_d4", "d3_d4_cycle", "d3_d4_magic_bias", "d5_d4_half_turn_ls", "d5_d4_half_turn_sollya",
            "d5_d4_half_turn_sollya_fast", "d5_d4", "d7_d6")
TOLERANCE = {"native": 1e-4, "d3_d4": 2e-4, "d3_d4_cycle": 2e-4, "d3_d4_magic_bias": 2e-4, "d5_d4_half_turn_ls": 1.4e-3,
             "d5_d4_half_turn_sollya": 7e-4, "d5_d4_half_turn_sollya_fast": 7e-4, "d5_d4": 3e-5, "d7_d6": 5e-7}


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def angles(n, seed, span):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-span, span, n).astype(np.float32)
    if n >= 16:
        a[:12] = [0.0, -0.0, math.pi / 4, -math.pi / 4, math.pi / 2, math.pi, -math.pi, 2 * math.pi, 1e-6, -1e-6, 100.5, -777.25]
    return a


def f32_bits(t):
    return t.detach().cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("variant", range(1, 9))
def test_sincos_f32_bit_exact_against_oracle(fpt, cuda, oracle, variant):
    import torch
    for n, span in ((0, 1.0), (1, 1.0), (3, 3.0), (1031, math.pi), ((1 << 18) + 3, 64.0), (1 << 16, 8192.0)):
        a = angles(n, seed=n + variant, span=span)
        ad = torch.from_numpy(a).to(cuda)
        out = torch.empty(2, n, dtype=torch.float32, device=cuda)
        fpt.call("fpt_sincos_f32", out.data_ptr(), ad.data_ptr(), n, variant, 0, stream())
        torch.cuda.synchronize()
        assert_bits_equal(f32_bits(out), oracle.sincos_f32(variant, a).view(np.uint32), f"{VARIANTS[variant]} n={n}")
        if n and span <= 64.0:
            tol = TOLERANCE[VARIANTS[variant]]
            assert np.abs(out[0].double().cpu().numpy() - np.cos(a.astype(np.float64))).max() < tol
            assert np.abs(out[1].double().cpu().numpy() - np.sin(a.astype(np.float64))).max() < tol


def test_sincos_f32_unaligned_views_and_probes(fpt, cuda, oracle):
    import torch
    n = 4099
    a = angles(n + 1, seed=9, span=20.0)
    ad = torch.from_numpy(a).to(cuda)
    out = torch.empty(2 * n + 8, dtype=torch.float32, device=cuda)
    # angle pointer off by one element: the all-scalar path
    fpt.call("fpt_sincos_f32", out.data_ptr(), ad.data_ptr() + 4, n, 7, 0, stream())
    torch.cuda.synchronize()
    assert_bits_equal(f32_bits(out[:2 * n]), oracle.sincos_f32(7, a[1:]).view(np.uint32).ravel(), "unaligned angles")
    for variant in (1, 2, 4, 6, 8):
        for iterations in (1, 5):
            o2 = torch.empty(2, n, dtype=torch.float32, device=cuda)
            fpt.call("fpt_sincos_f32", o2.data_ptr(), ad.data_ptr(), n, variant, iterations, stream())
            torch.cuda.synchronize()
            assert_bits_equal(f32_bits(o2), oracle.sincos_f32(variant, a[:n], iterations).view(np.uint32),
                              f"probe {VARIANTS[variant]} x{iterations}")


def test_sincos_f32_native_control_is_accurate(fpt, cuda):
    import torch
    a = angles(1 << 16, seed=4, span=math.pi)
    ad = torch.from_numpy(a).to(cuda)
    out = torch.empty(2, a.size, dtype=torch.float32, device=cuda)
    fpt.call("fpt_sincos_f32", out.data_ptr(), ad.data_ptr(), a.size, 0, 0, stream())
    torch.cuda.synchronize()
    assert np.abs(out[0].double().cpu().numpy() - np.cos(a.astype(np.float64))).max() < TOLERANCE["native"]
    assert np.abs(out[1].double().cpu().numpy() - np.sin(a.astype(np.float64))).max() < TOLERANCE["native"]


def test_sincos_f32_reference_kernels_agree(fpt, cuda, ref_kernels):
    """Bit for bit with the reference's compiled fp32 kernels (all eight polynomial variants, plain and probe)."""
    import torch
    n = 1 << 18
    problems = []
    for span in (math.pi, 8192.0):
        a = torch.from_numpy(angles(n, seed=5, span=span)).to(cuda)
        for variant in range(1, 9):
            ours = torch.empty(2, n, dtype=torch.float32, device=cuda)
            ref = torch.empty_like(ours)
            fpt.call("fpt_sincos_f32", ours.data_ptr(), a.data_ptr(), n, variant, 0, stream())
            torch.cuda.synchronize()
            ref_call(ref_kernels, f"launch_sincos_{VARIANTS[variant]}_f32", ref, a, n)
            torch.cuda.synchronize()
            bad = int((f32_bits(ours) != f32_bits(ref)).sum())
            if bad:
                problems.append(f"{VARIANTS[variant]} span {span}: {bad} of {2 * n} differ")
            fpt.call("fpt_sincos_f32", ours.data_ptr(), a.data_ptr(), n, variant, 3, stream())
            torch.cuda.synchronize()
            ref_call(ref_kernels, f"launch_sincos_{VARIANTS[variant]}_compute_f32", ref, a, n, 3)
            torch.cuda.synchronize()
            bad = int((f32_bits(ours) != f32_bits(ref)).sum())
            if bad:
                problems.append(f"{VARIANTS[variant]} probe span {span}: {bad} of {2 * n} differ")
    assert not problems, problems


def increments(head_dim, theta=500000.0):
    freqs = theta ** (-np.arange(0, head_dim, 2, dtype=np.float64) / head_dim)
    return np.round(freqs * (2.0 ** 32) / (2 * math.pi)).astype(np.int64).astype(np.uint32)


def test_rope_lut_table_bit_exact_accurate_and_like_the_reference(fpt, cuda, oracle, ref_kernels):
    import torch
    seq, head_dim = 1031, 128
    inc = increments(head_dim)
    incd = torch.from_numpy(inc.view(np.int32)).to(cuda)
    lut = oracle.rope_phase_table()
    lutd = torch.from_numpy(lut.view(np.int16).copy()).to(cuda).view(torch.float16)
    for iterations in (0, 4):
        table = torch.empty(2, seq, inc.size, dtype=torch.float16, device=cuda)
        fpt.call("fpt_rope_table_lut", table.data_ptr(), incd.data_ptr(), lutd.data_ptr(), seq, inc.size, iterations, stream())
        torch.cuda.synchronize()
        assert_bits_equal(to_bits(table), oracle.rope_table_lut(inc, lut, seq, iterations), f"rope lut x{iterations}")
        ref = torch.empty_like(table)
        if iterations:
            ref_call(ref_kernels, "launch_rope_sincos_fixed_lut_fp16_compute", ref, incd, lutd, seq, inc.size, iterations)
        else:
            ref_call(ref_kernels, "launch_rope_sincos_fixed_lut_fp16", ref, incd, lutd, seq, inc.size)
        torch.cuda.synchronize()
        assert_bits_equal(to_bits(table), to_bits(ref), f"reference rope lut x{iterations}")
        if not iterations:
            pos = np.arange(seq, dtype=np.float64)[:, None]
            ang = pos * (inc.astype(np.float64)[None, :] * 2 * math.pi / 2.0 ** 32)
            assert np.abs(table[0].double().cpu().numpy() - np.cos(ang)).max() < 2.5e-3
            assert np.abs(table[1].double().cpu().numpy() - np.sin(ang)).max() < 2.5e-3


def test_python_names_of_the_fp32_and_lut_ops(fpt, cuda, oracle):
    import torch
    from fast_polynomial_transcendentals_b200 import spline_ops
    a = angles(4096, seed=2, span=10.0)
    ad = torch.from_numpy(a).to(cuda).view(64, 64)
    out = spline_ops.sincos_d7_d6_f32(ad)
    assert out.shape == (2, 64, 64) and out.dtype == torch.float32
    assert_bits_equal(f32_bits(out).ravel(), oracle.sincos_f32("d7_d6", a).view(np.uint32).ravel(), "sincos_d7_d6_f32")
    probe = spline_ops.sincos_d3_d4_cycle_compute_f32(ad, 2)
    assert_bits_equal(f32_bits(probe).ravel(), oracle.sincos_f32("d3_d4_cycle", a, 2).view(np.uint32).ravel(), "cycle probe")
    with pytest.raises(RuntimeError, match="float32"):
        spline_ops.sincos_native_f32(ad.half())
    with pytest.raises(RuntimeError, match="positive"):
        spline_ops.sincos_d5_d4_compute_f32(ad, 0)
    inc = increments(64)
    incd = torch.from_numpy(inc.view(np.int32)).to(cuda)
    lut = oracle.rope_phase_table()
    lutd = torch.from_numpy(lut.view(np.int16).copy()).to(cuda).view(torch.float16)
    table = spline_ops.rope_sincos_fixed_lut_fp16(incd, lutd, 77)
    assert_bits_equal(to_bits(table), oracle.rope_table_lut(inc, lut, 77), "rope_sincos_fixed_lut_fp16")
    with pytest.raises(RuntimeError, match=r"\[128, 2\]"):
        spline_ops.rope_sincos_fixed_lut_fp16(incd, lutd[:64], 77)
