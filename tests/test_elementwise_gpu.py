"""GPU parity of the element-wise kernels: bit-exact against the CPU oracle and, where the
reference's own kernels were compiled into oracle/_ref, bit-exact against those too."""
import numpy as np
import pytest

from util import assert_bits_equal, normal_bits, ref_call, to_bits, to_device, uniform_bits

pytestmark = pytest.mark.gpu

DT = {"fp16": 0, "bf16": 1}
FN = {"SIGMOID": 0, "TANH": 1, "SWISH": 2, "ERF": 3, "GELU": 4}


def programs(oracle):
    return [(i, r) for i, r in enumerate(oracle.program_table()) if r["shape"] not in ("ALG_SIG", "ALG_TANH")]


def run_unary(fpt, cuda, row, bits, repeats=1):
    import torch
    dtype = "bf16" if row["dtype"] else "fp16"
    fn, direction, _ = row["name"].split("_")
    x = to_device(bits, dtype, cuda)
    out = torch.empty_like(x)
    fpt.call("fpt_unary_repeat", out.data_ptr(), x.data_ptr(), x.numel(), FN[fn], 0 if direction == "FWD" else 1,
             row["degree"], row["dtype"], row["source"], repeats, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return to_bits(out)


def test_every_program_is_bit_exact(fpt, cuda, oracle):
    """All 104 polynomial programs, 2^16 + 3 seeded inputs each (vector body + ragged tail)."""
    for idx, row in programs(oracle):
        dtype = "bf16" if row["dtype"] else "fp16"
        bits = uniform_bits((1 << 16) + 3, -10.0, 10.0, dtype, seed=100 + idx)
        assert_bits_equal(run_unary(fpt, cuda, row, bits), oracle.unary(idx, bits),
                          f'{row["name"]}/{dtype}/{row["source"]}', bits)


def test_every_16bit_pattern_primary_programs(fpt, cuda, oracle):
    """Exhaustive: all 65536 input patterns (every NaN payload, subnormal, infinity) for the deployed programs."""
    allbits = np.arange(65536, dtype=np.uint16)
    for name, dt in (("SIGMOID_FWD_D3", 0), ("TANH_FWD_D4", 0), ("SWISH_FWD_D3", 0), ("GELU_FWD_D5", 0),
                     ("SIGMOID_FWD_D3", 1), ("TANH_FWD_D4", 1), ("SWISH_FWD_D3", 1), ("SWISH_FWD_D5", 1)):
        idx = oracle.find_program(name, dt)
        row = oracle.program_table()[idx]
        assert_bits_equal(run_unary(fpt, cuda, row, allbits), oracle.unary(idx, allbits), f"{name}/{dt}", allbits)


@pytest.mark.parametrize("n", [0, 1, 2, 7, 8, 9, 31, 4095 * 2, 4096 * 2, 4096 * 2 + 5, (1 << 20) + 13])
def test_sizes_and_tails(fpt, cuda, oracle, n):
    idx = oracle.find_program("SIGMOID_FWD_D3", 0)
    row = oracle.program_table()[idx]
    bits = uniform_bits(n, -8.0, 8.0, "fp16", seed=n)
    assert_bits_equal(run_unary(fpt, cuda, row, bits), oracle.unary(idx, bits), f"n={n}", bits)


def test_misaligned_pointers_take_the_scalar_path(fpt, cuda, oracle):
    import torch
    idx = oracle.find_program("SWISH_FWD_D3", 1)
    bits = uniform_bits(10001, -8.0, 8.0, "bf16", seed=5)
    base = to_device(np.concatenate([np.zeros(3, np.uint16), bits]), "bf16", cuda)
    x = base[3:]                       # 6-byte offset: not 16-byte aligned
    outbase = torch.zeros(10001 + 1, dtype=torch.bfloat16, device=cuda)
    out = outbase[1:]
    fpt.call("fpt_unary", out.data_ptr(), x.data_ptr(), x.numel(), 2, 0, 3, 1, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert_bits_equal(to_bits(out), oracle.unary(idx, bits), "misaligned", bits)


def test_config1_style_inputs_streaming_regime(fpt, cuda, oracle):
    """2^24 bf16 values U[-16,16) with 1% specials through SWISH D3 (exercises the HBM-streaming variant
    when forced) and the default variant; both bit-exact."""
    idx = oracle.find_program("SWISH_FWD_D3", 1)
    row = oracle.program_table()[idx]
    bits = uniform_bits(1 << 24, -16.0, 16.0, "bf16")
    want = oracle.unary(idx, bits)
    for streaming in (-1, 1, 0):
        assert fpt.load().fpt_set_tuning(b"streaming", streaming) == 0
        try:
            assert_bits_equal(run_unary(fpt, cuda, row, bits), want, f"streaming={streaming}", bits)
        finally:
            fpt.load().fpt_set_tuning(b"streaming", -1)
    for blocks in (1, 8):
        assert fpt.load().fpt_set_tuning(b"blocks_per_sm", blocks) == 0
        try:
            assert_bits_equal(run_unary(fpt, cuda, row, bits), want, f"blocks_per_sm={blocks}", bits)
        finally:
            fpt.load().fpt_set_tuning(b"blocks_per_sm", 0)


def test_repeated_evaluation_probe(fpt, cuda, oracle):
    for name, dt in (("SIGMOID_FWD_D3", 0), ("TANH_FWD_D4", 1), ("SWISH_FWD_D3", 0)):
        idx = oracle.find_program(name, dt)
        row = oracle.program_table()[idx]
        bits = uniform_bits(5000, -8.0, 8.0, "bf16" if dt else "fp16", seed=9)
        for repeats in (2, 16):
            assert_bits_equal(run_unary(fpt, cuda, row, bits, repeats), oracle.unary(idx, bits, repeats),
                              f"{name} x{repeats}", bits)


def test_gradient_products(fpt, cuda, oracle):
    import torch
    for idx, row in programs(oracle):
        fn, direction, _ = row["name"].split("_")
        if direction != "BWD":
            continue
        dtype = "bf16" if row["dtype"] else "fp16"
        xb = uniform_bits(20011, -8.0, 8.0, dtype, seed=idx)
        gb = normal_bits(20011, 1.0, dtype, seed=idx + 1)
        x, go = to_device(xb, dtype, cuda), to_device(gb, dtype, cuda)
        gi = torch.empty_like(x)
        fpt.call("fpt_binary_bwd", gi.data_ptr(), go.data_ptr(), x.data_ptr(), x.numel(), FN[fn], row["degree"],
                 row["dtype"], row["source"], torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert_bits_equal(to_bits(gi), oracle.binary_bwd(idx, gb, xb), f'{row["name"]}/{dtype}/{row["source"]}', xb)


def test_algebraic_gradients(fpt, cuda, oracle):
    import torch
    for dt, dtype in ((0, "fp16"), (1, "bf16")):
        for fn, name in ((0, "SIGMOID_BWD_ALGEBRAIC"), (1, "TANH_BWD_ALGEBRAIC")):
            idx = oracle.find_program(name, dt)
            yb = uniform_bits(9999, -1.0, 1.0, dtype, seed=3)
            gb = normal_bits(9999, 1.0, dtype, seed=4)
            y, go = to_device(yb, dtype, cuda), to_device(gb, dtype, cuda)
            gi = torch.empty_like(y)
            fpt.call("fpt_bwd_algebraic", gi.data_ptr(), go.data_ptr(), y.data_ptr(), y.numel(), fn, dt,
                     torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert_bits_equal(to_bits(gi), oracle.binary_bwd(idx, gb, yb), name + dtype, yb)


def test_native_controls_are_close_to_the_true_function(fpt, cuda):
    import torch
    x = torch.linspace(-8, 8, 40001, device=cuda)
    for dtype, tol in ((torch.float16, 2e-3), (torch.bfloat16, 1.6e-2)):
        xi = x.to(dtype)
        for fn, true in ((0, torch.sigmoid), (1, torch.tanh), (2, torch.nn.functional.silu), (4, torch.nn.functional.gelu)):
            out = torch.empty_like(xi)
            fpt.call("fpt_unary", out.data_ptr(), xi.data_ptr(), xi.numel(), fn, 0, 0,
                     1 if dtype == torch.bfloat16 else 0, 0, torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            err = (out.float() - true(xi.float())).abs()
            scale = true(xi.float()).abs().clamp_min(1.0)
            assert float((err / scale).max()) < tol, (dtype, fn, float((err / scale).max()))


# ---- bit-exactness against the reference's own compiled kernels ------------------------------

REF_UNARY = [("sigmoid", 0), ("tanh", 1), ("swish", 2), ("gelu", 4)]


def test_reference_kernels_agree_bit_for_bit_unary(fpt, cuda, oracle, ref_kernels):
    import torch
    for fn_name, fn in REF_UNARY:
        for degree in (3, 4, 5, 6):
            for dtype, dt, suffixes in (("fp16", 0, [("", 0)]), ("bf16", 1, [("_bf16", 0), ("_bf16_sollya", 1)])):
                for suffix, source in suffixes:
                    bits = uniform_bits(1 << 18, -12.0, 12.0, dtype, seed=degree * 10 + dt)
                    x = to_device(bits, dtype, cuda)
                    ours, ref = torch.empty_like(x), torch.empty_like(x)
                    fpt.call("fpt_unary", ours.data_ptr(), x.data_ptr(), x.numel(), fn, 0, degree, dt, source,
                             torch.cuda.current_stream().cuda_stream)
                    symbol = f"launch_{fn_name}_fwd_d{degree}_kernel{suffix}"
                    if not hasattr(ref_kernels, symbol):
                        continue
                    torch.cuda.synchronize()
                    ref_call(ref_kernels, symbol, ref, x, x.numel())
                    torch.cuda.synchronize()
                    assert_bits_equal(to_bits(ours), to_bits(ref), symbol, bits)


def test_reference_kernels_agree_bit_for_bit_backward(fpt, cuda, ref_kernels):
    import torch
    for fn_name, fn in REF_UNARY:
        for degree in (3, 4, 5, 6):
            for dtype, dt, suffix in (("fp16", 0, ""), ("bf16", 1, "_bf16")):
                xb = uniform_bits(1 << 17, -10.0, 10.0, dtype, seed=degree)
                gb = normal_bits(1 << 17, 1.0, dtype, seed=degree + 50)
                x, go = to_device(xb, dtype, cuda), to_device(gb, dtype, cuda)
                ours, ref = torch.empty_like(x), torch.empty_like(x)
                fpt.call("fpt_binary_bwd", ours.data_ptr(), go.data_ptr(), x.data_ptr(), x.numel(), fn, degree, dt, 0,
                         torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                symbol = f"launch_{fn_name}_bwd_d{degree}_kernel{suffix}"
                ref_call(ref_kernels, symbol, ref, go, x, x.numel())
                torch.cuda.synchronize()
                assert_bits_equal(to_bits(ours), to_bits(ref), symbol, xb)
