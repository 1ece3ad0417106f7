"""GPU: tensor-core building blocks and the attention forward against the fp32 CPU oracle."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_umma_tile_matches_matmul(fpt, cuda, mode):
    """One 128^3 bf16 tile: Q K^T form (both operands K-major), P V form (tensor-memory A, MN-major B) and the dQ form
    (A stored by the threads into swizzled shared memory and read MN-major, B MN-major)."""
    import torch
    g = torch.Generator(device=cuda)
    g.manual_seed(1234 + mode)
    a = torch.randn(128, 128, device=cuda, generator=g).to(torch.bfloat16)
    b = torch.randn(128, 128, device=cuda, generator=g).to(torch.bfloat16)
    c = torch.full((128, 128), float("nan"), device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    fpt.call("fpt_selftest_umma", c.data_ptr(), a.data_ptr(), b.data_ptr(), mode, status.data_ptr(), stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 0, hex(int(status.item()) & 0xFFFFFFFF)
    want = (a.float() @ b.float().t()) if mode == 0 else (a.float() @ b.float()) if mode == 1 else (a.float().t() @ b.float())
    err = (c - want).abs().max().item()
    assert err < 1e-3 * max(1.0, want.abs().max().item()), err


def run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap=0.0, log2_n=12, exp2_emu_freq=None, exp2_emu_backend=0):
    """q,k,v torch bf16 (B,S,H,D), any strides with D contiguous. Returns (out (B,S,Hq,D), lse, status)."""
    import ctypes
    import torch
    B, S, Hq, D = q.shape
    Hk = k.shape[2]
    out = torch.full((B, S, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    lse = torch.full((B, Hq, S), float("nan"), dtype=torch.float32, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    if exp2_emu_freq is None:
        fpt.call("fpt_attention_fwd", out.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, Hq, Hk,
                 D, arr(q), arr(k), arr(v), arr(out), mode, int(causal), scale, softcap, log2_n, status.data_ptr(), stream())
    else:
        fpt.call("fpt_attention_fwd_routed", out.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S,
                 Hq, Hk, D, arr(q), arr(k), arr(v), arr(out), mode, int(causal), scale, softcap, log2_n, exp2_emu_backend,
                 exp2_emu_freq, status.data_ptr(), stream())
    torch.cuda.synchronize()
    return out, lse, int(status.item()) & 0xFFFFFFFF


def bits(t):
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


UNNORMALISED = (1, 4)     # sigmoid attention (polynomial, special-function unit): O = P V without a row sum


class Tolerance:
    """Accumulates |got - want| over the (batch, head) blocks of one case and judges it by the mode.

    Soft-max modes: 2e-2 max-abs on the bf16 output (rows are convex combinations of V, so values are of order one).
    Sigmoid modes: the output is a plain sum with probabilities of order 1/n, its size shrinks like 1/sqrt(n) (standard
    deviation 0.12 at 512 keys, 0.02 at 16384), so an absolute bound says nothing there: per block the largest error
    must stay within 2e-2 of the block's largest value, and over the whole case the mean error within 5e-3 of the mean
    magnitude."""

    def __init__(self, mode):
        self.unnormalised = mode in UNNORMALISED
        self.worst_abs = self.worst_rel = self.sum_err = self.sum_ref = 0.0

    def add(self, got, want):
        err = np.abs(got.astype(np.float64) - want.astype(np.float64))
        self.worst_abs = max(self.worst_abs, float(err.max()))
        self.worst_rel = max(self.worst_rel, float(err.max()) / max(float(np.abs(want).max()), 1e-30))
        self.sum_err += float(err.sum())
        self.sum_ref += float(np.abs(want).sum())

    def check(self, what=""):
        if self.unnormalised:
            assert self.worst_rel <= 2e-2, (what, "largest error relative to the block's largest value", self.worst_rel)
            assert self.sum_err <= 5e-3 * self.sum_ref, (what, "relative mean error", self.sum_err / max(self.sum_ref, 1e-30))
        else:
            assert self.worst_abs <= 2e-2, (what, self.worst_abs)


CASES = [
    # (B, S, Hq, Hk, mode, causal, softcap, log2_n)
    (1, 128, 1, 1, 2, False, 0.0, 12),
    (1, 256, 2, 1, 2, True, 0.0, 12),
    (1, 384, 4, 2, 0, True, 50.0, 12),
    (2, 512, 4, 1, 0, True, 30.0, 12),
    (1, 512, 2, 2, 1, False, 0.0, 9),
    (1, 384, 2, 1, 1, True, 0.0, 12),
    (1, 1024, 8, 2, 0, True, 50.0, 12),
    # sequence lengths that are not multiples of the 128-key tile (ragged last tile, zero-filled and masked)
    (1, 200, 2, 1, 2, True, 0.0, 12),
    (2, 333, 4, 2, 0, False, 30.0, 12),
    (1, 77, 1, 1, 1, False, 0.0, 12),
    (1, 257, 2, 2, 1, True, 0.0, 12),
    (1, 130, 2, 1, 2, False, 0.0, 12),
    # a single position, and one key more than two tiles
    (1, 1, 2, 1, 2, True, 0.0, 12),
    (1, 1, 1, 1, 0, False, 50.0, 12),
    (1, 257, 4, 1, 0, True, 50.0, 12),
    # the native twins of the two score-mods: tanh.approx soft-cap (both layouts: cap 50 column-split, cap 100 not) and
    # the ex2 + rcp sigmoid, against the oracle's exact tanh / exact sigmoid
    (1, 384, 4, 2, 3, True, 50.0, 12),
    (2, 333, 4, 2, 3, False, 30.0, 12),
    (1, 640, 2, 1, 3, True, 100.0, 12),
    (1, 1, 1, 1, 3, False, 50.0, 12),
    (1, 512, 2, 2, 4, False, 0.0, 9),
    (1, 384, 2, 1, 4, True, 0.0, 12),
    (1, 77, 1, 1, 4, False, 0.0, 7),
    (1, 2048, 2, 1, 4, False, 0.0, 11),
]


@pytest.mark.parametrize("case", CASES)
def test_attention_matches_fp32_oracle(fpt, cuda, oracle, case):
    """Output against the fp32 CPU attention that uses the same score-mod: 2e-2 max-abs for the soft-max modes, bounds
    relative to the signal for the unnormalised sigmoid modes (class Tolerance)."""
    import torch
    B, S, Hq, Hk, mode, causal, softcap, log2_n = case
    D = 128
    g = torch.Generator(device=cuda)
    g.manual_seed(1234)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    out, lse, status = run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    assert status == 0, hex(status)
    assert not torch.isnan(out.float()).any()
    qb, kb, vb = bits(q), bits(k), bits(v)
    rng = np.random.default_rng(7)
    tol = Tolerance(mode)
    for b in range(B):
        for h in range(Hq):
            rows = np.arange(S) if (b == 0 and h in (0, Hq - 1)) else np.sort(rng.choice(S, size=min(S, 32), replace=False))
            want = oracle.attention_rows(qb, kb, vb, b, h, rows, mode, causal, scale, softcap, log2_n)
            tol.add(out[b, rows, h, :].float().cpu().numpy(), want)
    tol.check(case)


PAIR_CASES = [
    # two query heads of one K / V group per pair of CTAs (causal and not), every mode and both soft-cap layouts
    (1, 1024, 4, 2, 2, True, 0.0, 12), (2, 640, 4, 1, 2, False, 0.0, 12), (1, 1024, 4, 2, 0, True, 30.0, 12),
    (1, 1024, 4, 2, 0, True, 100.0, 12), (1, 768, 8, 2, 1, True, 0.0, 12), (1, 1024, 4, 2, 3, True, 30.0, 12),
    (1, 512, 2, 1, 4, False, 0.0, 9), (1, 1000, 4, 1, 2, True, 0.0, 12), (1, 333, 2, 1, 0, False, 50.0, 12),
    # two neighbouring row blocks of one head (no K / V sharing between heads, no mask)
    (2, 1024, 2, 2, 1, False, 0.0, 10), (1, 2048, 3, 3, 2, False, 0.0, 12), (1, 1024, 1, 1, 0, False, 50.0, 12),
    # blocks that cannot pair (one head per K / V head under a causal mask; an odd number of row blocks): the call falls
    # back to single CTAs
    (1, 1024, 2, 2, 2, True, 0.0, 12), (1, 768, 3, 3, 1, False, 0.0, 12),
]


@pytest.mark.parametrize("case", PAIR_CASES)
def test_pairs_of_ctas_give_the_same_bits(fpt, cuda, case):
    """`attention_cta_pair` = 1 runs the forward on clusters of two CTAs (one 256-row product for two SMs, K and V tiles
    split between them): same products, same order, so output and log-sum-exp are the single-CTA kernel's bit for bit."""
    import torch
    B, S, Hq, Hk, mode, causal, softcap, log2_n = case
    D = 128
    g = torch.Generator(device=cuda)
    g.manual_seed(99)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    base, lse0, status = run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    assert status == 0, hex(status)
    fpt.call("fpt_set_tuning", b"attention_cta_pair", 1)
    try:
        got, lse1, status = run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    finally:
        fpt.call("fpt_set_tuning", b"attention_cta_pair", 0)
    assert status == 0, hex(status)
    assert torch.equal(base.view(torch.int16), got.view(torch.int16))
    if mode not in UNNORMALISED:
        assert torch.equal(lse0.view(torch.int32), lse1.view(torch.int32))


def test_attention_accepts_head_major_layout(fpt, cuda):
    """(B,H,S,D) storage (what the fused RoPE writes) addressed through strides gives the same result."""
    import torch
    B, S, H, D = 1, 256, 2, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(5)
    q = torch.randn(B, S, H, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, H, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    ref, _, st0 = run_attention(fpt, cuda, q, k, v, 2, True, scale)
    qh = q.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)   # same values, (B,H,S,D) memory
    kh = k.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    alt, _, st1 = run_attention(fpt, cuda, qh, kh, v, 2, True, scale)
    assert st0 == 0 and st1 == 0
    assert torch.equal(ref.view(torch.int16), alt.view(torch.int16))


def test_plain_softmax_mode_matches_torch_sdpa(fpt, cuda):
    import torch
    B, S, Hq, Hk, D = 1, 512, 4, 2, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(11)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    out, lse, status = run_attention(fpt, cuda, q, k, v, 2, True, 1.0 / math.sqrt(D))
    assert status == 0
    kk = k.repeat_interleave(Hq // Hk, dim=2)
    vv = v.repeat_interleave(Hq // Hk, dim=2)
    want = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2).float(), kk.transpose(1, 2).float(), vv.transpose(1, 2).float(), is_causal=True).transpose(1, 2)
    assert float((out.float() - want).abs().max()) < 2e-2
    scores = torch.einsum("bshd,bthd->bhst", q.float(), kk.float()) / math.sqrt(D)
    mask = torch.ones(S, S, device=cuda, dtype=torch.bool).tril()
    want_lse = torch.logsumexp(scores.masked_fill(~mask, float("-inf")), dim=-1)
    assert float((lse - want_lse).abs().max()) < 1e-2


@pytest.mark.parametrize("freq", [8, 12, 16, 32])
@pytest.mark.parametrize("mode,causal,softcap", [(2, True, 0.0), (0, True, 30.0), (2, False, 0.0)])
def test_routed_exp2_stays_within_tolerance(fpt, cuda, oracle, freq, mode, causal, softcap):
    """Four of every `freq` keys take the fp32 cubic exponential: same 2e-2 bound against the fp32 oracle, and
    within bf16 rounding of the unrouted kernel."""
    import torch
    B, S, Hq, Hk, D = 1, 384, 2, 1, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(99)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    base, lse0, st0 = run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap, 12, exp2_emu_freq=0)
    out, lse, st = run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap, 12, exp2_emu_freq=freq)
    assert st0 == 0 and st == 0
    # the two differ by a rounding flip of the bf16 output at most: one unit in the last place of the value
    assert bool(((out.float() - base.float()).abs() <= 0.0079 * base.float().abs().clamp(min=1.0)).all())
    assert float((lse - lse0).abs().max()) < 1e-3
    qb, kb, vb = bits(q), bits(k), bits(v)
    rows = np.arange(S)
    for h in range(Hq):
        want = oracle.attention_rows(qb, kb, vb, 0, h, rows, mode, causal, scale, softcap, 12)
        assert float(np.abs(out[0, :, h, :].float().cpu().numpy() - want).max()) < 2e-2


FULL_SIZE = [
    # the two attention workloads of the benchmark, at their full sizes: (B, S, Hq, Hk, mode, causal, softcap, log2_n)
    ("causal GQA, soft-cap 50", 4, 8192, 32, 8, 0, True, 50.0, 12),
    ("sigmoid, bidirectional", 2, 16384, 32, 32, 1, False, 0.0, 14),
]


@pytest.mark.parametrize("case", FULL_SIZE, ids=[c[0] for c in FULL_SIZE])
def test_full_size_workloads_by_sampled_rows_and_properties(fpt, cuda, oracle, case):
    """At the benchmark's sizes the oracle cannot redo everything, but a row of attention costs it only S x D: sampled
    rows of sampled heads against the fp32 oracle (bounds of class Tolerance), plus two properties that need no oracle.  Causal: rows before
    position p do not change by a bit when keys and values from p on are replaced.  Both modes: the output is linear in
    V, so O(V) + O(V') agrees with O(V + V') up to the bf16 roundings of the three outputs."""
    import torch
    _, B, S, Hq, Hk, mode, causal, softcap, log2_n = case
    D = 128
    g = torch.Generator(device=cuda)
    g.manual_seed(4242)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    out, lse, status = run_attention(fpt, cuda, q, k, v, mode, causal, scale, softcap, log2_n)
    assert status == 0 and not torch.isnan(out.float()).any()
    qb, kb, vb = bits(q), bits(k), bits(v)
    rng = np.random.default_rng(11)
    tol = Tolerance(mode)
    for b in range(B):
        for h in range(0, Hq, 8):      # every 8th head of every batch entry, 64 rows each (a row costs the oracle S x D)
            rows = np.unique(np.concatenate([[0, 1, 127, 128, S - 129, S - 1], rng.choice(S, size=58, replace=False)]))
            want = oracle.attention_rows(qb, kb, vb, b, h, rows, mode, causal, scale, softcap, log2_n)
            tol.add(out[b, rows, h, :].float().cpu().numpy(), want)
    tol.check(case[0])
    if causal:
        cut = S // 2 + 37
        k2, v2 = k.clone(), v.clone()
        k2[:, cut:] = torch.randn(B, S - cut, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
        v2[:, cut:] = torch.randn(B, S - cut, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
        out2, lse2, status2 = run_attention(fpt, cuda, q, k2, v2, mode, causal, scale, softcap, log2_n)
        assert status2 == 0
        assert torch.equal(out[:, :cut], out2[:, :cut]) and torch.equal(lse[:, :, :cut], lse2[:, :, :cut])
        assert not torch.equal(out[:, cut:], out2[:, cut:])
        del k2, v2, out2, lse2
    v_other = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v_sum = (v.float() + v_other.float()).to(torch.bfloat16)
    out_other, _, st1 = run_attention(fpt, cuda, q, k, v_other, mode, causal, scale, softcap, log2_n)
    out_sum, _, st2 = run_attention(fpt, cuda, q, k, v_sum, mode, causal, scale, softcap, log2_n)
    assert st1 == 0 and st2 == 0
    # the sum of V itself is rounded to bf16 (relative 2^-9 per element) before it is averaged by the probabilities
    residual = (out.float() + out_other.float() - out_sum.float()).abs().max()
    assert float(residual) < 3e-2 * float(out_sum.float().abs().max()), float(residual)


@pytest.mark.parametrize("freq", [8, 32])
def test_routed_two_piece_exponential(fpt, cuda, oracle, freq):
    """Backend "pwl2" (2 % exponential) on a share of the lanes: outputs stay within a bound that scales with the share."""
    import torch
    B, S, Hq, Hk, D = 1, 384, 2, 1, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(98)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    base, lse0, st0 = run_attention(fpt, cuda, q, k, v, 2, True, scale, 0.0, 12, exp2_emu_freq=0)
    out, lse, st = run_attention(fpt, cuda, q, k, v, 2, True, scale, 0.0, 12, exp2_emu_freq=freq, exp2_emu_backend=1)
    assert st0 == 0 and st == 0
    diff = float((out.float() - base.float()).abs().max())
    lse_diff = float((lse - lse0).abs().max())
    assert diff < 0.03 * 4 / freq * 8 + 8e-3, diff
    assert lse_diff < 0.03, lse_diff
    with pytest.raises(Exception):      # the two-piece line is offered for the plain soft-max only
        run_attention(fpt, cuda, q, k, v, 0, True, scale, 30.0, 12, exp2_emu_freq=freq, exp2_emu_backend=1)


@pytest.mark.parametrize("backend,name,err,oracle_bound", [(2, "d2_safe", 2.7e-3, 2e-2), (3, "pwl2_safe_f16", 1.14e-2, 3.5e-2)])
@pytest.mark.parametrize("freq", [12, 32])
def test_routed_endpoint_preserving_exponentials(fpt, cuda, oracle, backend, name, err, oracle_bound, freq):
    """The two retained routed backends of the reference (forward frequency 12): outputs stay within 2e-2 of the
    fp32 oracle (3.5e-2 for the fp16 line, whose own error is 1.1e-2 on the routed weights) and within the evaluator's
    error plus two bf16 roundings of the all-SFU kernel;
    rows that rescale several times (scores growing along the sequence) stay finite and within the same bound, which is
    what the endpoint constraints p(0) = 1, p(1) = 2 are for."""
    import torch
    B, S, Hq, Hk, D = 1, 640, 2, 1, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(97)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g) * torch.linspace(0.3, 5.0, S, device=cuda).view(1, S, 1, 1)
    q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    qb, kb, vb = bits(q), bits(k), bits(v)
    for causal in (True, False):
        base, lse0, st0 = run_attention(fpt, cuda, q, k, v, 2, causal, scale, 0.0, 12, exp2_emu_freq=0)
        out, lse, st = run_attention(fpt, cuda, q, k, v, 2, causal, scale, 0.0, 12, exp2_emu_freq=freq, exp2_emu_backend=backend)
        assert st0 == 0 and st == 0 and not torch.isnan(out.float()).any()
        assert not torch.equal(out, base), "the routed kernel must not be the unrouted one"
        assert float((lse - lse0).abs().max()) < 2 * err
        # the evaluator's error on the routed weights plus one bf16 rounding of each of the two outputs
        largest = max(1.0, float(base.float().abs().max()))
        assert float((out.float() - base.float()).abs().max()) < (1.2 * err + 2.0 ** -7) * largest
        for h in range(Hq):
            want = oracle.attention_rows(qb, kb, vb, 0, h, np.arange(S), 2, causal, scale, 0.0, 12)
            assert float(np.abs(out[0, :, h, :].float().cpu().numpy() - want).max()) < oracle_bound, (name, freq, causal)
    with pytest.raises(Exception):      # offered for the plain soft-max only
        run_attention(fpt, cuda, q, k, v, 0, True, scale, 30.0, 12, exp2_emu_freq=freq, exp2_emu_backend=backend)


def test_routed_exp2_rejects_unbuilt_frequencies(fpt, cuda):
    import torch
    q = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device=cuda)
    for mode, freq in ((2, 4), (2, 10), (2, -8), (1, 12), (3, 8), (4, 8)):
        with pytest.raises(Exception):
            run_attention(fpt, cuda, q, q, q, mode, False, 1.0, 0.0, 12, exp2_emu_freq=freq)


def test_running_maximum_that_keeps_growing_is_rescaled(fpt, cuda, oracle):
    """Keys whose scores grow along the sequence force the lazy rescale (maximum up by more than 2^8 between tiles)
    several times per row; a second block of rows sees it shrink again."""
    import torch
    B, S, Hq, Hk, D = 1, 1024, 2, 1, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(3)
    q = torch.randn(B, S, Hq, D, device=cuda, generator=g)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g)
    ramp = torch.linspace(0.2, 6.0, S, device=cuda).view(1, S, 1, 1)
    k = k * ramp                                    # later keys reach far larger scores
    k[:, S // 2:, :, :] *= torch.linspace(1.0, 0.1, S // 2, device=cuda).view(1, -1, 1, 1)
    q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    qb, kb, vb = bits(q), bits(k), bits(v)
    rows = np.arange(S)
    for causal in (False, True):
        for freq in (0, 12):
            out, lse, st = run_attention(fpt, cuda, q, k, v, 2, causal, scale, 0.0, 12, exp2_emu_freq=freq)
            assert st == 0
            assert not torch.isnan(out.float()).any()
            for h in range(Hq):
                want = oracle.attention_rows(qb, kb, vb, 0, h, rows, 2, causal, scale, 0.0, 12)
                assert float(np.abs(out[0, :, h, :].float().cpu().numpy() - want).max()) < 2e-2


@pytest.mark.parametrize("softcap,gain", [(50.0, 1.0), (50.0, 12.0), (30.0, 30.0), (100.0, 1.0), (100.0, 12.0),
                                          (0.5, 1.0), (67.5, 40.0), (67.5, 1.0)])   # the ends of the column-split range
def test_softcap_layouts_and_saturating_scores(fpt, cuda, oracle, softcap, gain):
    """Soft-cap 30 / 50 take the column-split layout with its fixed exponent reference, 100 the one-thread-per-row
    layout with a running maximum; `gain` pushes most scores into the saturated part of the tanh program (rows whose
    first tile sits at -cap while later tiles reach +cap are the reference's worst case)."""
    import torch
    B, S, Hq, Hk, D = 1, 640, 2, 1, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(2024)
    q = (torch.randn(B, S, Hq, D, device=cuda, generator=g) * gain).to(torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device=cuda, generator=g)
    k[:, :128] = -k[:, :128].abs() * torch.sign(q[:, :1, :1, :].float().mean(dim=2, keepdim=True))   # a hostile first tile
    k = k.to(torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device=cuda, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    qb, kb, vb = bits(q), bits(k), bits(v)
    rows = np.arange(S)
    for causal in (False, True):
        results = []
        for split in (1, 0):
            assert fpt.load().fpt_set_tuning(b"attention_split", split) == 0
            out, lse, status = run_attention(fpt, cuda, q, k, v, 0, causal, scale, softcap, 12)
            assert status == 0 and not torch.isnan(out.float()).any() and not torch.isnan(lse).any()
            results.append((out, lse))
        assert fpt.load().fpt_set_tuning(b"attention_split", 1) == 0
        # the two layouts round P against different exponent references: both must sit within the tolerance of the
        # oracle, and their log-sum-exp (not rounded to bf16) must agree closely
        assert float((results[0][1] - results[1][1]).abs().max()) < 2e-3, "lse of the two layouts"
        for h in range(Hq):
            want = oracle.attention_rows(qb, kb, vb, 0, h, rows, 0, causal, scale, softcap, 12)
            for out, _ in results:
                err = float(np.abs(out[0, :, h, :].float().cpu().numpy() - want).max())
                assert err < 2e-2, (softcap, gain, causal, h, err)


def test_bounded_wait_runs_out_and_later_blocks_skip(fpt, cuda):
    """The bounded mbarrier wait of the attention kernels, on a barrier nobody arrives on (one thread, no TMA, no tensor
    memory, nothing in flight): it gives up after the limit, records 0x80000000 | where in the status word, and a block
    started afterwards finds the word set and does not wait at all."""
    import torch
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    report = torch.zeros(3, dtype=torch.int32, device=cuda)
    limit_ns, where = 200_000, 7
    fpt.call("fpt_selftest_bounded_wait", status.data_ptr(), report.data_ptr(), limit_ns, where, stream())
    torch.cuda.synchronize()
    r = report.cpu().numpy().view(np.uint32)
    waited = int(r[1]) | (int(r[2]) << 32)
    assert int(status.item()) & 0xFFFFFFFF == 0x80000000 | where
    assert int(r[0]) == 1, "the wait must have timed out"
    assert limit_ns <= waited < 50 * limit_ns, waited       # gave up after the limit, and soon after it
    report.zero_()
    fpt.call("fpt_selftest_bounded_wait", status.data_ptr(), report.data_ptr(), limit_ns, where + 1, stream())
    torch.cuda.synchronize()
    r = report.cpu().numpy().view(np.uint32)
    assert int(r[0]) == 2 and int(r[1]) == 0, "a block that starts after a timeout must skip its work at once"
    assert int(status.item()) & 0xFFFFFFFF == 0x80000000 | where    # the first report is kept
    for bad in (0, 999, 1_000_001):
        assert fpt.load().fpt_selftest_bounded_wait(status.data_ptr(), report.data_ptr(), bad, where, stream()) == -2
    # the context is intact: a tensor-core self-test right afterwards passes
    a = torch.randn(128, 128, device=cuda).to(torch.bfloat16)
    c = torch.empty(128, 128, device=cuda)
    ok = torch.zeros(1, dtype=torch.int32, device=cuda)
    fpt.call("fpt_selftest_umma", c.data_ptr(), a.data_ptr(), a.data_ptr(), 0, ok.data_ptr(), stream())
    torch.cuda.synchronize()
    assert int(ok.item()) == 0 and float((c - a.float() @ a.float().t()).abs().max()) < 1e-3 * float(c.abs().max())
