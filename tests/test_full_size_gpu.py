"""GPU: the element-wise workloads at the benchmark's full sizes.

The oracle cannot redo 2^28 elements in a test, so parity at these sizes goes through properties that do not depend on
the size:
  * a unary program is a function of one 16-bit pattern: the full-size output must equal, element by element, a table of
    the program on all 65536 patterns, and that table is compared with the oracle bit for bit;
  * for two-input and fp32-input kernels, a million seeded positions (plus the first and last elements) are redone by
    the oracle, and the packed and flat layouts of SwiGLU must agree bit for bit over the whole tensor.
"""
import math

import numpy as np
import pytest

from util import assert_bits_equal

pytestmark = pytest.mark.gpu

N_FULL = 1 << 28


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def table_lookup_equal(torch, table_i16, x_i16, out_i16, chunk=1 << 26):
    """out[i] == table[x[i]] for every i, in chunks (the index tensor is 8 bytes per element)."""
    for start in range(0, x_i16.numel(), chunk):
        idx = x_i16[start:start + chunk].to(torch.int64) & 0xFFFF
        if not torch.equal(table_i16[idx], out_i16[start:start + chunk]):
            bad = torch.nonzero(table_i16[idx] != out_i16[start:start + chunk])[:4].flatten().tolist()
            return False, [start + b for b in bad]
    return True, []


@pytest.mark.parametrize("name,fn,degree", [("SIGMOID_FWD_D3", 0, 3), ("TANH_FWD_D4", 1, 4), ("SWISH_FWD_D3", 2, 3)])
def test_unary_programs_at_2_to_28(fpt, cuda, oracle, name, fn, degree):
    import torch
    g = torch.Generator(device=cuda)
    g.manual_seed(28)
    x = (torch.rand(N_FULL, device=cuda, generator=g) * 16 - 8).to(torch.float16)
    x.view(torch.int16)[::4093] = torch.arange(0, (N_FULL + 4092) // 4093, device=cuda).to(torch.int16)   # 65585 values: every pattern occurs
    out = torch.empty_like(x)
    fpt.call("fpt_unary", out.data_ptr(), x.data_ptr(), N_FULL, fn, 0, degree, 0, 0, stream())
    patterns = torch.arange(65536, device=cuda).to(torch.int16).view(torch.float16)
    table = torch.empty_like(patterns)
    fpt.call("fpt_unary", table.data_ptr(), patterns.data_ptr(), 65536, fn, 0, degree, 0, 0, stream())
    torch.cuda.synchronize()
    allbits = np.arange(65536, dtype=np.uint16)
    assert_bits_equal(table.view(torch.int16).cpu().numpy().view(np.uint16), oracle.unary(oracle.find_program(name, 0), allbits),
                      f"{name} table", allbits)
    ok, where = table_lookup_equal(torch, table.view(torch.int16), x.view(torch.int16), out.view(torch.int16))
    assert ok, where


@pytest.mark.parametrize("variant", [1, 0])
def test_exp2_fraction_at_2_to_28(fpt, cuda, oracle, variant):
    import torch
    g = torch.Generator(device=cuda)
    g.manual_seed(29)
    x = torch.rand(N_FULL, device=cuda, generator=g).to(torch.float16).clamp_(max=0.9995)
    out = torch.empty_like(x)
    fpt.call("fpt_exp2_fraction", out.data_ptr(), x.data_ptr(), N_FULL, variant, 1, stream())
    patterns = torch.arange(65536, device=cuda).to(torch.int16).view(torch.float16)
    table = torch.empty_like(patterns)
    fpt.call("fpt_exp2_fraction", table.data_ptr(), patterns.data_ptr(), 65536, variant, 1, stream())
    torch.cuda.synchronize()
    if variant == 1:       # the hinge polynomial has an oracle; the native control is only checked for self-consistency
        allbits = np.arange(65536, dtype=np.uint16)
        assert_bits_equal(table.view(torch.int16).cpu().numpy().view(np.uint16), oracle.exp2_hinge(allbits, 0), "hinge table", allbits)
    ok, where = table_lookup_equal(torch, table.view(torch.int16), x.view(torch.int16), out.view(torch.int16))
    assert ok, where


def test_sincos_at_2_to_28_sampled_positions(fpt, cuda, oracle):
    import torch
    g = torch.Generator(device=cuda)
    g.manual_seed(30)
    a = torch.rand(N_FULL, device=cuda, generator=g) * (2 * math.pi) - math.pi
    out = torch.empty(2, N_FULL, dtype=torch.int16, device=cuda)
    fpt.call("fpt_sincos", out.data_ptr(), a.data_ptr(), N_FULL, 3, 0, stream())
    torch.cuda.synchronize()
    rng = np.random.default_rng(31)
    pos = np.unique(np.concatenate([[0, 1, 7, N_FULL - 8, N_FULL - 1], rng.integers(0, N_FULL, size=1 << 20)]))
    idx = torch.from_numpy(pos).to(cuda)
    want_c, want_s = oracle.sincos_packed(3, a[idx].cpu().numpy())
    assert_bits_equal(out[0][idx].cpu().numpy().view(np.uint16), want_c, "cos at sampled positions")
    assert_bits_equal(out[1][idx].cpu().numpy().view(np.uint16), want_s, "sin at sampled positions")


@pytest.mark.parametrize("rows,hidden", [(16384, 14336), (131072, 1408)], ids=["B1_dense", "B4_routed"])
def test_swiglu_full_size_layouts_agree_and_samples_match(fpt, cuda, oracle, rows, hidden):
    import torch
    g = torch.Generator(device=cuda)
    g.manual_seed(32)
    packed = (torch.randn(rows, 2 * hidden, device=cuda, generator=g) * 1.5).to(torch.bfloat16)
    gate, up = packed[:, :hidden].contiguous(), packed[:, hidden:].contiguous()
    flat = torch.empty_like(gate)
    from_packed = torch.empty_like(gate)
    fpt.call("fpt_swish_mul", flat.data_ptr(), gate.data_ptr(), up.data_ptr(), rows * hidden, 3, 1, 0, stream())
    fpt.call("fpt_swish_mul_packed", from_packed.data_ptr(), packed.data_ptr(), rows, hidden, 3, 1, 0, stream())
    torch.cuda.synchronize()
    assert torch.equal(flat.view(torch.int16), from_packed.view(torch.int16))
    rng = np.random.default_rng(33)
    n = rows * hidden
    pos = np.unique(np.concatenate([[0, 1, hidden - 1, hidden, n - hidden, n - 1], rng.integers(0, n, size=1 << 20)]))
    idx = torch.from_numpy(pos).to(cuda)
    bits_of = lambda t: t.reshape(-1)[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.swiglu(oracle.find_program("SWISH_FWD_D3", 1, 0), bits_of(gate), bits_of(up))
    assert_bits_equal(bits_of(flat), want, "SwiGLU at sampled positions")


def test_rope_prologue_at_the_sigmoid_attention_size(fpt, cuda, oracle):
    """B=2, S=16384, 32 heads, D=128, theta = 500000, bf16 in and out: the whole tensor against the oracle (its phase
    arithmetic is integer, so position 16383 is as exact as position 0)."""
    import torch
    B, S, H, D = 2, 16384, 32, 128
    freqs = 500000.0 ** (-np.arange(0, D, 2, dtype=np.float64) / D)
    inc = np.round(freqs / (2 * math.pi) * 2.0 ** 32).astype(np.uint64).astype(np.uint32)
    incd = torch.from_numpy(inc.view(np.int32)).to(cuda)
    g = torch.Generator(device=cuda)
    g.manual_seed(34)
    q = torch.randn(B, S, H, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, H, D, device=cuda, generator=g).to(torch.bfloat16)
    qo = torch.empty(B, H, S, D, dtype=q.dtype, device=cuda)
    ko = torch.empty_like(qo)
    fpt.call("fpt_rope_apply", qo.data_ptr(), ko.data_ptr(), q.data_ptr(), k.data_ptr(), incd.data_ptr(), B, S, H, H, D, 0, 1,
             stream())
    torch.cuda.synchronize()
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    import os
    oracle.set_threads(os.cpu_count() or 1)
    want_q, want_k = oracle.rope_apply(bits(q), bits(k), inc, io_bf16=True)
    assert np.array_equal(bits(qo), want_q)
    assert np.array_equal(bits(ko), want_k)
