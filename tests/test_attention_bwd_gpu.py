"""GPU: attention backward (dQ, dK, dV) of the three modes against the float64 CPU restatement that uses the same
polynomial score-mods, and plain softmax against torch autograd."""
import ctypes
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def bits(t):
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def forward(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n):
    import torch
    B, S, Hq, D = q.shape
    out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.zeros(B, Hq, S, dtype=torch.float32, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    fpt.call("fpt_attention_fwd", out.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, Hq,
             k.shape[2], D, arr(q), arr(k), arr(v), arr(out), mode, int(causal), scale, softcap, log2_n, status.data_ptr(), stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out, lse


def backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, softcap, log2_n, softcap_grad=0, emu=None, single_pass=False):
    import torch
    B, S, Hq, D = q.shape
    Hk = k.shape[2]
    dq = torch.full((B, S, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    dk = torch.full((B, S, Hk, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    dv = torch.full((B, S, Hk, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    need = fpt.load().fpt_attention_bwd_workspace_bytes(B, S, Hq)
    assert need == 2 * B * Hq * ((S + 127) // 128 * 128) * 4
    if single_pass:      # the planes plus the fp32 dQ buffer: the entry point then takes its one-pass form
        need = fpt.load().fpt_attention_bwd_fused_workspace_bytes(B, S, Hq)
        assert need == 2 * B * Hq * ((S + 127) // 128 * 128) * 4 + B * S * Hq * D * 4
    workspace = torch.full((need,), 0x7F, dtype=torch.uint8, device=cuda)       # garbage: the entry point clears what it needs
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    if emu is None:
        fpt.call("fpt_attention_bwd", dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(), k.data_ptr(),
                 v.data_ptr(), out.data_ptr(), lse.data_ptr(), workspace.data_ptr(), need, B, S, Hq, Hk, D, arr(q), arr(k), arr(v),
                 arr(out), arr(dout), mode, int(causal), scale, softcap, log2_n, softcap_grad, status.data_ptr(), stream())
    else:           # (backend, frequency) of the software exponential
        fpt.call("fpt_attention_bwd_routed", dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(),
                 k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), workspace.data_ptr(), need, B, S, Hq, Hk, D, arr(q),
                 arr(k), arr(v), arr(out), arr(dout), mode, int(causal), scale, softcap, log2_n, softcap_grad, emu[0], emu[1],
                 status.data_ptr(), stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 0, hex(int(status.item()) & 0xFFFFFFFF)
    return dq, dk, dv


def close(got, want, what, rel=2e-2):
    import torch
    g = got.float().cpu().numpy().astype(np.float64)
    assert not np.isnan(g).any(), what
    err = np.abs(g - want).max()
    assert err <= rel * max(np.abs(want).max(), 1e-6), (what, err, np.abs(want).max())


CASES = [
    # (B, S, Hq, Hk, mode, causal, softcap, log2_n, softcap_grad)
    (1, 128, 1, 1, 2, False, 0.0, 12, 0),
    (1, 256, 2, 1, 2, True, 0.0, 12, 0),
    (2, 384, 4, 2, 2, True, 0.0, 12, 0),
    (1, 384, 4, 2, 0, True, 50.0, 12, 0),
    (1, 256, 2, 2, 0, False, 30.0, 12, 1),
    (1, 512, 2, 1, 1, False, 0.0, 9, 0),
    (1, 384, 4, 2, 1, True, 0.0, 12, 0),
    # ragged sequence lengths
    (1, 200, 2, 1, 2, True, 0.0, 12, 0),
    (2, 333, 4, 2, 0, False, 30.0, 12, 0),
    (1, 77, 1, 1, 1, False, 0.0, 12, 0),
    (1, 257, 4, 2, 2, False, 0.0, 12, 0),
    (1, 130, 2, 1, 1, True, 0.0, 12, 0),
    # the native twins: tanh on the special-function unit with 1 - t^2, exact sigmoid with p (1 - p)
    (1, 384, 4, 2, 3, True, 50.0, 12, 1),
    (2, 333, 4, 2, 3, False, 30.0, 12, 1),
    (1, 256, 2, 1, 3, True, 100.0, 12, 1),
    (1, 512, 2, 1, 4, False, 0.0, 9, 0),
    (1, 384, 4, 2, 4, True, 0.0, 12, 0),
    (1, 77, 1, 1, 4, False, 0.0, 7, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_backward_matches_the_cpu_restatement(fpt, cuda, oracle, case):
    import torch
    from oracle import attention_bwd
    B, S, Hq, Hk, mode, causal, softcap, log2_n, softcap_grad = case
    D = 128
    g = torch.Generator(device=cuda)
    g.manual_seed(4321)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    dout = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    out, lse = forward(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    dq, dk, dv = backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, softcap, log2_n, softcap_grad)
    _, _, want_dq, want_dk, want_dv = attention_bwd.attention_fwd_bwd(bits(q), bits(k), bits(v), bits(dout), mode, causal, scale,
                                                                      softcap, log2_n, softcap_grad)
    close(dq, want_dq, "dq")
    close(dk, want_dk, "dk")
    close(dv, want_dv, "dv")


@pytest.mark.parametrize("backend,freq,bound", [(0, 8, 2e-2), (0, 32, 2e-2), (2, 12, 2e-2), (2, 32, 2e-2), (3, 12, 3e-2),
                                                (3, 32, 2e-2), (1, 16, 5e-2)])
def test_backward_with_routed_software_exponential(fpt, cuda, backend, freq, bound):
    """Four of every `freq` columns recompute their probability with a software exponential (cubic 8.8e-5, quadratic
    2.7e-3, fp16 two-piece line 1.1e-2, two-piece line 2.1e-2 relative): gradients stay within the bound of the float64
    restatement, relative to the largest gradient, and differ from the unrouted kernel (the route is taken)."""
    import torch
    from oracle import attention_bwd
    B, S, Hq, Hk, D = 1, 384, 4, 2, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(2468)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    dout = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    for causal in (True, False):
        out, lse = forward(fpt, cuda, q, k, v, 2, causal, scale, 0.0, 12)
        base = backward(fpt, cuda, q, k, v, out, lse, dout, 2, causal, scale, 0.0, 12, emu=(backend, 0))
        dq, dk, dv = backward(fpt, cuda, q, k, v, out, lse, dout, 2, causal, scale, 0.0, 12, emu=(backend, freq))
        _, _, want_dq, want_dk, want_dv = attention_bwd.attention_fwd_bwd(bits(q), bits(k), bits(v), bits(dout), 2, causal, scale)
        close(dq, want_dq, "dq", bound)
        close(dk, want_dk, "dk", bound)
        close(dv, want_dv, "dv", bound)
        assert not torch.equal(dv, base[2]), "the routed kernel must not be the unrouted one"
    lib = fpt.load()
    t = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device=cuda)
    ws = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    arr = (ctypes.c_int64 * 3)(128 * 128, 128, 128)
    lse1 = torch.zeros(1, 1, 128, device=cuda)
    common = lambda mode, be, fr: lib.fpt_attention_bwd_routed(
        t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
        lse1.data_ptr(), ws.data_ptr(), 4096, 1, 128, 1, 1, 128, arr, arr, arr, arr, arr, mode, 0, 1.0, 30.0, 12, 0, be, fr,
        st.data_ptr(), None)
    assert common(2, 0, 10) == -5 and common(2, 9, 8) == -5      # unknown frequency, unknown backend
    assert common(0, 0, 8) == -5 and common(1, 0, 8) == -5       # routed for the plain soft-max only


@pytest.mark.parametrize("case", CASES)
def test_single_pass_backward_matches_the_cpu_restatement_and_the_two_pass_form(fpt, cuda, oracle, case):
    """The one-pass form (dK / dV blocks also produce the partial dQ tiles, added in fp32; 5 matrix products instead of
    7; the default when the workspace holds the fp32 dQ buffer): same tolerance against the float64 restatement; dK and dV are the same bits as the two-pass form (same
    arithmetic, same order); dQ differs from it by the rounding of one fp32 sum at most (one bf16 unit in the last place
    of the largest gradients)."""
    import torch
    from oracle import attention_bwd
    B, S, Hq, Hk, mode, causal, softcap, log2_n, softcap_grad = case
    D = 128
    g = torch.Generator(device=cuda)
    g.manual_seed(4321)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    dout = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    out, lse = forward(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    # the smaller workspace selects the two-pass form, the larger one the single-pass form (tuning key at its default, 1)
    two = backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, softcap, log2_n, softcap_grad)
    lib = fpt.load()
    value = ctypes.c_int(-1)
    assert lib.fpt_get_tuning(b"attention_bwd_fused", ctypes.byref(value)) == 0 and value.value == 1
    one = backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, softcap, log2_n, softcap_grad, single_pass=True)
    _, _, want_dq, want_dk, want_dv = attention_bwd.attention_fwd_bwd(bits(q), bits(k), bits(v), bits(dout), mode, causal, scale,
                                                                      softcap, log2_n, softcap_grad)
    close(one[0], want_dq, "dq")
    close(one[1], want_dk, "dk")
    close(one[2], want_dv, "dv")
    assert torch.equal(one[1], two[1]) and torch.equal(one[2], two[2]), "dK / dV of the two forms must be the same bits"
    gap = (one[0].float() - two[0].float()).abs().max()
    assert float(gap) <= 2.0 ** -7 * float(two[0].float().abs().max()), float(gap)
    # tuning key 2: the same kernel with sixteen score-mod warps per block instead of eight: dK and dV the same bits again
    assert lib.fpt_set_tuning(b"attention_bwd_fused", 2) == 0
    try:
        wide = backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, softcap, log2_n, softcap_grad, single_pass=True)
    finally:
        assert lib.fpt_set_tuning(b"attention_bwd_fused", 1) == 0
    close(wide[0], want_dq, "dq, sixteen score-mod warps")
    assert torch.equal(wide[1], two[1]) and torch.equal(wide[2], two[2])
    # with the tuning key off the same call, large workspace and all, takes the two-pass form: bits equal
    assert lib.fpt_set_tuning(b"attention_bwd_fused", 0) == 0
    try:
        forced = backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, softcap, log2_n, softcap_grad, single_pass=True)
    finally:
        assert lib.fpt_set_tuning(b"attention_bwd_fused", 1) == 0
    assert all(torch.equal(a, b) for a, b in zip(forced, two))


def test_plain_softmax_backward_matches_torch_autograd(fpt, cuda):
    import torch
    B, S, Hq, Hk, D = 1, 512, 4, 2, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(77)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    dout = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    out, lse = forward(fpt, cuda, q, k, v, 2, True, scale, 0.0, 12)
    dq, dk, dv = backward(fpt, cuda, q, k, v, out, lse, dout, 2, True, scale, 0.0, 12)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    kk = kf.repeat_interleave(Hq // Hk, dim=2)
    vv = vf.repeat_interleave(Hq // Hk, dim=2)
    ref = torch.nn.functional.scaled_dot_product_attention(qf.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                           is_causal=True).transpose(1, 2)
    ref.backward(dout.float())
    for got, want, name in ((dq, qf.grad, "dq"), (dk, kf.grad, "dk"), (dv, vf.grad, "dv")):
        err = float((got.float() - want).abs().max())
        assert err <= 2e-2 * float(want.abs().max()), (name, err)


def test_backward_rejects_bad_arguments(fpt, cuda):
    import torch
    lib = fpt.load()
    t = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device=cuda)
    lse = torch.zeros(1, 1, 128, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    ws = torch.zeros(2048, dtype=torch.uint8, device=cuda)
    arr = (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))

    def call(workspace_bytes=1024, mode=2, seq=128, out=t.data_ptr()):
        return lib.fpt_attention_bwd(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                     t.data_ptr(), out, lse.data_ptr(), ws.data_ptr(), workspace_bytes, 1, seq, 1, 1, 128,
                                     arr, arr, arr, arr, arr, mode, 0, 1.0, 1.0, 12, 0, status.data_ptr(), None)

    assert call(workspace_bytes=8) == -9                 # workspace too small
    assert call(mode=7) < 0
    assert call(out=None) < 0                            # soft-max modes need the forward output
    assert call(mode=1, out=None, workspace_bytes=0) == 0   # the sigmoid mode needs neither out, lse nor workspace
    torch.cuda.synchronize()


@pytest.mark.parametrize("mode,causal", [(2, True), (1, False), (0, True)])
def test_block_order_does_not_change_a_bit(fpt, cuda, mode, causal):
    """The two hand-out orders of the blocks (tuning key "attention_raster") run the same per-block work: forward and
    backward results are identical bit for bit; the sigmoid-mode column-split layout (attention_split 2) likewise."""
    import torch
    B, S, Hq, Hk, D = 2, 600, 4, 2, 128           # ragged: 600 is not a multiple of the tile
    g = torch.Generator(device=cuda)
    g.manual_seed(31)
    mk = lambda h: torch.randn(B, S, h, D, device=cuda, generator=g).to(torch.bfloat16)
    q, k, v, dout = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
    scale = 1.0 / math.sqrt(D)
    lib = fpt.load()
    results = []
    try:
        for raster, split in ((0, 1), (1, 1), (-1, 2)):
            assert lib.fpt_set_tuning(b"attention_raster", raster) == 0
            assert lib.fpt_set_tuning(b"attention_split", split) == 0
            out, lse = forward(fpt, cuda, q, k, v, mode, causal, scale, 30.0, 10)
            dq, dk, dv = backward(fpt, cuda, q, k, v, out, lse, dout, mode, causal, scale, 30.0, 10)
            results.append((out, dq, dk, dv) + (() if mode == 1 else (lse,)))
    finally:
        assert lib.fpt_set_tuning(b"attention_raster", -1) == 0
        assert lib.fpt_set_tuning(b"attention_split", 1) == 0
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert torch.equal(a, b)
    value = ctypes.c_int(7)
    assert lib.fpt_get_tuning(b"attention_raster", ctypes.byref(value)) == 0 and value.value == -1
    assert lib.fpt_set_tuning(b"attention_raster", 2) != 0


def test_full_size_backward_properties(fpt, cuda):
    """The benchmark's causal GQA soft-cap workload at full size (B=4, S=8192, 32 / 8 heads), where the float64
    restatement is out of reach: the gradients are linear in dO (same probabilities, same polynomial derivative), and dQ
    of the rows before position p does not change by a bit when keys and values from p on are replaced."""
    import torch
    B, S, Hq, Hk, D = 4, 8192, 32, 8, 128
    mode, causal, softcap, log2_n = 0, True, 50.0, 12
    g = torch.Generator(device=cuda)
    g.manual_seed(99)
    mk = lambda h: torch.randn(B, S, h, D, device=cuda, generator=g).to(torch.bfloat16)
    q, k, v, d1, d2 = mk(Hq), mk(Hk), mk(Hk), mk(Hq), mk(Hq)
    scale = 1.0 / math.sqrt(D)
    out, lse = forward(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    d12 = (d1.float() + d2.float()).to(torch.bfloat16)
    g1 = backward(fpt, cuda, q, k, v, out, lse, d1, mode, causal, scale, softcap, log2_n)
    g2 = backward(fpt, cuda, q, k, v, out, lse, d2, mode, causal, scale, softcap, log2_n)
    g12 = backward(fpt, cuda, q, k, v, out, lse, d12, mode, causal, scale, softcap, log2_n)
    for a, b_, c, what in zip(g1, g2, g12, ("dq", "dk", "dv")):
        assert not torch.isnan(c.float()).any(), what
        top = float(c.float().abs().max())
        residual = float((a.float() + b_.float() - c.float()).abs().max())
        assert residual < 3e-2 * top, (what, residual, top)
    cut = S // 2 + 37
    k2, v2 = k.clone(), v.clone()
    k2[:, cut:] = mk(Hk)[:, cut:]
    v2[:, cut:] = mk(Hk)[:, cut:]
    out2, lse2 = forward(fpt, cuda, q, k2, v2, mode, causal, scale, softcap, log2_n)
    dq2, _, _ = backward(fpt, cuda, q, k2, v2, out2, lse2, d1, mode, causal, scale, softcap, log2_n)
    assert torch.equal(g1[0][:, :cut], dq2[:, :cut])
    assert not torch.equal(g1[0][:, cut:], dq2[:, cut:])
