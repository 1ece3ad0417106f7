"""GPU: the RoPE entry point for callers that cannot allocate device memory.

Some users of this library run where `cudaMalloc` is off limits: a plugin called inside a serving loop whose host
process owns every byte of device memory, a latency-critical path that must not touch the allocator, or a program
with no device allocator of its own.  The cached-table RoPE needs a [2, seq, head_dim/2] table between its two
kernels; `fpt_rope_apply_static_table` keeps that table in a fixed array inside the library instead of asking the
caller for it.  This test calls it through the C ABI twice in a row and checks both results bit for bit against
the ordinary route (fpt_rope_table into a caller-allocated table, then fpt_rope_apply with that table), and checks
that a problem larger than the fixed array is refused with a clear status.
"""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def increments(head_dim, theta=500000.0):
    freqs = theta ** (-np.arange(0, head_dim, 2, dtype=np.float64) / head_dim)
    return np.round(freqs * (2.0 ** 32) / (2 * math.pi)).astype(np.int64).astype(np.uint32)


def test_static_table_route_equals_the_allocating_route_twice(fpt, cuda):
    import torch
    lib = fpt.load()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fpt_rope_static_table_capacity() == 1 << 21
    g = torch.Generator(device=cuda)
    g.manual_seed(99)
    # different shapes, dtypes and table programs back to back: a call must not see anything left by the one before;
    # the third fills the fixed array to its last entry (16384 x 128 = 2^21)
    cases = (((2, 1024, 4, 2, 128), torch.float16, 0, 0), ((1, 300, 3, 1, 64), torch.bfloat16, 1, 1),
             ((1, 16384, 1, 1, 128), torch.float16, 0, 1), ((1, 512, 2, 2, 128), torch.bfloat16, 1, 0))
    for (B, S, Hq, Hk, D), dtype, dt, table_kind in cases:
        inc = torch.from_numpy(increments(D).view(np.int32)).to(cuda)
        q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(dtype)
        k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(dtype)
        table = torch.empty(2, S, D // 2, dtype=torch.float16, device=cuda)
        want_q = torch.empty(B, Hq, S, D, dtype=dtype, device=cuda)
        want_k = torch.empty(B, Hk, S, D, dtype=dtype, device=cuda)
        fpt.call("fpt_rope_table", table.data_ptr(), inc.data_ptr(), S, D // 2, table_kind, 0, stream)
        fpt.call("fpt_rope_apply", want_q.data_ptr(), want_k.data_ptr(), q.data_ptr(), k.data_ptr(), table.data_ptr(),
                 B, S, Hq, Hk, D, 3, dt, stream)
        got_q = torch.full_like(want_q, float("nan"))
        got_k = torch.full_like(want_k, float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(cuda)
        fpt.call("fpt_rope_apply_static_table", got_q.data_ptr(), got_k.data_ptr(), q.data_ptr(), k.data_ptr(),
                 inc.data_ptr(), B, S, Hq, Hk, D, table_kind, dt, stream)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(cuda)
        assert free_after == free_before, "the call must not take device memory from the driver"
        assert torch.equal(got_q.view(torch.int16), want_q.view(torch.int16))
        assert torch.equal(got_k.view(torch.int16), want_k.view(torch.int16))


def test_static_table_route_refuses_what_does_not_fit(fpt, cuda):
    import torch
    lib = fpt.load()
    p = torch.zeros(64, dtype=torch.int32, device=cuda).data_ptr()
    too_long = (1 << 21) // 128 + 8
    status = lib.fpt_rope_apply_static_table(p, p, p, p, p, 1, too_long, 1, 1, 128, 0, 0, None)
    assert status == -9
    assert b"scratch" in lib.fpt_status_string(status)


def test_static_table_route_checks_everything_before_it_enqueues(fpt, cuda):
    """Calls with a null or misaligned tensor, no increments, or an unknown table program or dtype are refused with the
    status of the failing check (the entry point runs every check of both of its steps before it enqueues the table
    kernel), and a valid call afterwards gives the same bits as before them."""
    import torch
    lib = fpt.load()
    stream = torch.cuda.current_stream().cuda_stream
    B, S, H, D = 1, 256, 2, 128
    inc = torch.from_numpy(increments(D).view(np.int32)).to(cuda)
    other = torch.from_numpy(increments(D, theta=10000.0).view(np.int32)).to(cuda)
    q = torch.randn(B, S, H, D, device=cuda).to(torch.float16)
    out_q, out_k = torch.empty(B, H, S, D, dtype=torch.float16, device=cuda), torch.empty(B, H, S, D, dtype=torch.float16, device=cuda)
    args = lambda qo, ko, qi, ki, params, kind=0, dt=0: (qo, ko, qi, ki, params, B, S, H, H, D, kind, dt, stream)
    fpt.call("fpt_rope_apply_static_table", *args(out_q.data_ptr(), out_k.data_ptr(), q.data_ptr(), q.data_ptr(), inc.data_ptr()))
    torch.cuda.synchronize()
    first = out_q.clone()
    ptr = q.data_ptr()
    assert lib.fpt_rope_apply_static_table(*args(None, out_k.data_ptr(), ptr, ptr, other.data_ptr())) == -1       # null output
    assert lib.fpt_rope_apply_static_table(*args(out_q.data_ptr(), out_k.data_ptr(), ptr + 2, ptr, other.data_ptr())) == -3  # misaligned q
    assert lib.fpt_rope_apply_static_table(*args(out_q.data_ptr(), out_k.data_ptr(), ptr, ptr, None)) == -1      # no increments
    assert lib.fpt_rope_apply_static_table(*args(out_q.data_ptr(), out_k.data_ptr(), ptr, ptr, other.data_ptr(), kind=2)) == -5
    assert lib.fpt_rope_apply_static_table(*args(out_q.data_ptr(), out_k.data_ptr(), ptr, ptr, other.data_ptr(), dt=4)) == -5
    torch.cuda.synchronize()
    fpt.call("fpt_rope_apply_static_table", *args(out_q.data_ptr(), out_k.data_ptr(), q.data_ptr(), q.data_ptr(), inc.data_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(out_q, first)
