"""GPU: the launch_* entry points of libfpt_b200_compat.so, called exactly as the reference's torch-facing C++ calls
them (reference: autonumerics_zero/spline_ops/spline_ops.cpp:14-288), against the reference's own compiled kernels
under the same names."""
import ctypes
import math
from pathlib import Path

import numpy as np
import pytest

from util import assert_bits_equal, normal_bits, ref_call, to_bits, to_device, uniform_bits

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def compat():
    return ctypes.CDLL(str(ROOT / "fast_polynomial_transcendentals_b200" / "libfpt_b200_compat.so"))


def test_same_symbols_same_bits(compat, cuda, ref_kernels):
    """One call per signature family through both libraries with identical arguments."""
    import torch
    n = 1 << 16
    problems = []

    def both(symbol, outputs, *args):
        mine = [torch.zeros_like(o) for o in outputs]
        theirs = [torch.zeros_like(o) for o in outputs]
        ref_call(compat, symbol, *mine, *args)
        ref_call(ref_kernels, symbol, *theirs, *args)
        torch.cuda.synchronize()
        assert compat.fpt_compat_last_status() == 0, symbol
        for a, b in zip(mine, theirs):
            if not torch.equal(a.view(torch.int16) if a.dtype != torch.float32 else a.view(torch.int32),
                               b.view(torch.int16) if b.dtype != torch.float32 else b.view(torch.int32)):
                problems.append(symbol)

    for dtype, suffixes in (("fp16", [""]), ("bf16", ["_bf16", "_bf16_sollya"])):
        x = to_device(uniform_bits(n, -9.0, 9.0, dtype, seed=1, special_fraction=0.0), dtype, cuda)
        go = to_device(normal_bits(n, 1.0, dtype, seed=2), dtype, cuda)
        up = to_device(normal_bits(n, 1.5, dtype, seed=3), dtype, cuda)
        for suffix in suffixes:
            both(f"launch_sigmoid_fwd_d3_kernel{suffix}", [x], x, n)
            both(f"launch_gelu_fwd_d5_kernel{suffix}", [x], x, n)
            both(f"launch_swish_bwd_d4_kernel{suffix}", [x], go, x, n)
            both(f"launch_swish_mul_fwd_d3_kernel{suffix}", [x], x, up, n)
            both(f"launch_swish_mul_bwd_d3_kernel{suffix}", [x, x], go, x, up, n)
            rows, hidden = 64, 512
            packed = torch.cat([x[: rows * hidden].view(rows, hidden), up[: rows * hidden].view(rows, hidden)], dim=1).contiguous()
            both(f"launch_swish_mul_packed_fwd_d3_kernel{suffix}", [x[: rows * hidden]], packed, rows, hidden)
            both(f"launch_swish_mul_packed_bwd_d4_kernel{suffix}", [packed], go[: rows * hidden].contiguous(), packed, rows, hidden)
        if dtype == "bf16":
            both("launch_sigmoid_bwd_alg_kernel_bf16", [x], go, x, n)
    x = to_device(uniform_bits(n, -9.0, 9.0, "fp16", seed=4, special_fraction=0.0), "fp16", cuda)
    go = to_device(normal_bits(n, 1.0, "fp16", seed=5), "fp16", cuda)
    both("launch_sigmoid_fused_kernel", [x, x], x, go, n)
    both("launch_swish_fwd_deriv_kernel", [x, x], x, n)
    both("launch_swish_fwd_hybrid_kernel", [x], x, n)
    both("launch_multiply_kernel", [x], x, go, n)
    ang = torch.from_numpy(np.random.default_rng(6).uniform(-50, 50, n).astype(np.float32)).to(cuda)
    both("launch_sincos_d7_d6_f32", [torch.empty(2, n, dtype=torch.float32, device=cuda)], ang, n)
    both("launch_sincos_d5_d4_compute_f32", [torch.empty(2, n, dtype=torch.float32, device=cuda)], ang, n, 3)
    both("launch_sincos_d5_d6_half_turn_fp16", [torch.empty(2, n, dtype=torch.float16, device=cuda)], ang, n)
    both("launch_sincos_d5_d6_half_turn_bf16_compute", [torch.empty(2, n, dtype=torch.bfloat16, device=cuda)], ang, n, 2)
    head_dim, seq = 128, 257
    freqs = 500000.0 ** (-np.arange(0, head_dim, 2, dtype=np.float64) / head_dim)
    inc = torch.from_numpy(np.round(freqs * 2.0 ** 32 / (2 * math.pi)).astype(np.int64).astype(np.uint32).view(np.int32)).to(cuda)
    table = torch.empty(2, seq, head_dim // 2, dtype=torch.float16, device=cuda)
    both("launch_rope_sincos_fixed_half_turn_d5_d6_fp16", [table], inc, seq, head_dim // 2)
    both("launch_rope_sincos_fixed_d3_d4_fp16_compute", [table], inc, seq, head_dim // 2, 3)
    B, Hq, Hk = 2, 4, 2
    q = torch.randn(B, seq, Hq, head_dim, device=cuda).half()
    k = torch.randn(B, seq, Hk, head_dim, device=cuda).half()
    q_out = torch.empty(B, Hq, seq, head_dim, dtype=torch.float16, device=cuda)
    k_out = torch.empty(B, Hk, seq, head_dim, dtype=torch.float16, device=cuda)
    both("launch_rope_apply_fixed_half_turn_d5_d6_fp16", [q_out, k_out], q, k, inc, B, seq, Hq, Hk, head_dim)
    assert not problems, problems


def test_rejected_arguments_are_reported_through_the_status_call(compat, cuda):
    import torch
    x = torch.zeros(64, dtype=torch.float16, device=cuda)
    ref_call(compat, "launch_sigmoid_fwd_d3_kernel", x, x, -5)
    assert compat.fpt_compat_last_status() < 0
    assert compat.fpt_compat_last_status() == 0          # reading clears it
    ang = torch.zeros(64, dtype=torch.float32, device=cuda)
    out = torch.zeros(2, 64, dtype=torch.float32, device=cuda)
    ref_call(compat, "launch_sincos_d3_d4_compute_f32", out, ang, 64, 0)   # a probe needs at least one evaluation
    assert compat.fpt_compat_last_status() < 0
