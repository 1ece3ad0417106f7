"""GPU parity of the gate / up projection with the SwiGLU in its epilogue (`fpt_gate_up_swiglu`).

Three statements, each at both tile heights:
  1. the products (`FPT_GATE_UP_RAW`) agree with an fp32 matrix product of the same bf16 inputs to bf16 rounding;
  2. the fused output equals the packed SwiGLU kernel applied to those products, bit for bit, and equals the CPU oracle's
     SwiGLU program on them, bit for bit: the epilogue IS the B1 / B4 program, only its operands never reach memory;
  3. grouped problems (empty groups, ragged ends, rows nobody owns) write exactly the rows their groups own.
"""
import ctypes

import numpy as np
import pytest

from util import assert_bits_equal, to_bits

pytestmark = pytest.mark.gpu

VP = ctypes.c_void_p


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def gate_up(fpt, x, wg, wu, ends=None, degree=3, raw=False, fill=float("nan")):
    import torch
    rows, dim = x.shape
    grouped = wg.dim() == 3
    hidden = wg.shape[-2]
    width = 2 * hidden if raw else hidden
    out = torch.full((rows, width), fill, dtype=torch.bfloat16, device=x.device)
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    fpt.call("fpt_gate_up_swiglu", out.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), rows, dim, hidden, x.stride(0),
             wg.stride(-2), wg.stride(0) if grouped else 0, width, VP(ends.data_ptr()) if ends is not None else None,
             wg.shape[0] if grouped else 1, degree, 0, 1 if raw else 0, status.data_ptr(), stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 0, hex(int(status.item()) & 0xFFFFFFFF)
    return out


def make(cuda, rows, dim, hidden, groups=1, seed=0):
    import torch
    g = torch.Generator(device=cuda)
    g.manual_seed(seed)
    x = torch.randn(rows, dim, device=cuda, generator=g).mul_(1.5).to(torch.bfloat16)
    shape = (hidden, dim) if groups == 1 else (groups, hidden, dim)
    wg = (torch.randn(*shape, device=cuda, generator=g) * dim ** -0.5).to(torch.bfloat16)
    wu = (torch.randn(*shape, device=cuda, generator=g) * dim ** -0.5).to(torch.bfloat16)
    return x, wg, wu


def products_fp32(x, wg, wu, ends=None):
    import torch
    hidden = wg.shape[-2]
    if ends is None:
        return torch.cat([x.float() @ wg.float().T, x.float() @ wu.float().T], dim=1)
    want = torch.zeros(x.shape[0], 2 * hidden, device=x.device)
    begin = 0
    for gi, end in enumerate(ends.tolist()):
        want[begin:end, :hidden] = x[begin:end].float() @ wg[gi].float().T
        want[begin:end, hidden:] = x[begin:end].float() @ wu[gi].float().T
        begin = end
    return want


@pytest.fixture(params=[(0, -1, 0), (128, -1, 0), (256, -1, 0), (0, 1, 1), (0, 0, 0)],
                ids=["auto", "tile_128", "tile_256", "cta_pair_wide", "one_cta"])
def tile_rows(request, fpt):
    """Every form of the kernel: the default (pairs of CTAs, one hidden tile per row tile), the two tile heights on one CTA,
    pairs with two hidden tiles per row tile (where their number is even), and single CTAs with the height left to the
    library (256 rows dense, 128 grouped)."""
    rows, pair, wide = request.param
    fpt.call("fpt_set_tuning", b"gate_up_tile_rows", rows)
    fpt.call("fpt_set_tuning", b"gate_up_cta_pair", pair)
    fpt.call("fpt_set_tuning", b"gate_up_pair_wide", wide)
    yield request.param
    fpt.call("fpt_set_tuning", b"gate_up_tile_rows", 0)
    fpt.call("fpt_set_tuning", b"gate_up_cta_pair", -1)
    fpt.call("fpt_set_tuning", b"gate_up_pair_wide", 0)


@pytest.mark.parametrize("rows,dim,hidden", [(1, 64, 128), (128, 64, 128), (300, 4096, 384), (1000, 200, 128), (777, 1024, 1408)])
def test_dense_products_and_epilogue(fpt, cuda, oracle, tile_rows, rows, dim, hidden):
    import torch
    x, wg, wu = make(cuda, rows, dim, hidden, seed=rows)
    raw = gate_up(fpt, x, wg, wu, raw=True)
    want = products_fp32(x, wg, wu)
    # fp32 accumulation in another order, then one rounding to bf16 (2^-9 relative): 2^-7 of the largest product bounds both
    assert float((raw.float() - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())
    rel = float((raw.float() - want).norm() / want.norm())
    assert rel < 3e-3, rel
    for degree in (3, 0):
        fused = gate_up(fpt, x, wg, wu, degree=degree)
        packed = torch.empty(rows, hidden, dtype=torch.bfloat16, device=cuda)
        fpt.call("fpt_swish_mul_packed", packed.data_ptr(), raw.data_ptr(), rows, hidden, degree, 1, 0, stream())
        torch.cuda.synchronize()
        assert_bits_equal(to_bits(fused), to_bits(packed), f"fused vs packed kernel on the raw products, degree {degree}")
    idx = oracle.find_program("SWISH_FWD_D3", 1, 0)
    bits = to_bits(raw)
    want_bits = oracle.swiglu(idx, np.ascontiguousarray(bits[:, :hidden]).ravel(), np.ascontiguousarray(bits[:, hidden:]).ravel())
    assert_bits_equal(to_bits(gate_up(fpt, x, wg, wu)).ravel(), want_bits, "fused vs the oracle's SwiGLU on the raw products")


def test_packed_weight_and_strided_views(fpt, cuda, tile_rows):
    """A packed [2 hidden, dim] weight passed as two views, and an x with a row stride larger than its width."""
    import torch
    rows, dim, hidden = 520, 512, 256
    x, wg, wu = make(cuda, rows, dim, hidden, seed=3)
    w = torch.cat([wg, wu], dim=0)
    wide = torch.zeros(rows, dim + 64, dtype=torch.bfloat16, device=cuda)
    wide[:, :dim] = x
    base = gate_up(fpt, x, wg, wu)
    assert torch.equal(gate_up(fpt, x, w[:hidden], w[hidden:]), base)
    assert torch.equal(gate_up(fpt, wide[:, :dim], wg, wu), base)


@pytest.mark.parametrize("ends", [[0, 0, 700, 700, 1500], [130, 131, 131, 900, 2000], [2000], [0, 0, 0]])
def test_grouped_rows_follow_their_group(fpt, cuda, tile_rows, ends):
    import torch
    rows, dim, hidden = 2000, 256, 256
    groups = len(ends)
    x, wg, wu = make(cuda, rows, dim, hidden, groups=groups, seed=len(ends))
    if groups == 1:
        wg, wu = wg.unsqueeze(0).contiguous(), wu.unsqueeze(0).contiguous()
    ends_t = torch.tensor(ends, dtype=torch.int32, device=cuda)
    raw = gate_up(fpt, x, wg, wu, ends_t, raw=True, fill=7.0)
    fused = gate_up(fpt, x, wg, wu, ends_t, fill=7.0)
    last = ends[-1]
    want = products_fp32(x, wg, wu, ends_t)
    if last:
        assert float((raw[:last].float() - want[:last]).abs().max()) <= 2.0 ** -7 * float(want.abs().max())
        packed = torch.empty(last, hidden, dtype=torch.bfloat16, device=cuda)
        fpt.call("fpt_swish_mul_packed", packed.data_ptr(), raw[:last].contiguous().data_ptr(), last, hidden, 3, 1, 0, stream())
        torch.cuda.synchronize()
        assert torch.equal(fused[:last], packed)
    # rows past the last end belong to no group: untouched
    assert bool((raw[last:] == 7.0).all()) and bool((fused[last:] == 7.0).all())


def test_forms_agree_bit_for_bit(fpt, cuda):
    """One CTA with either tile height and a pair of CTAs add the same products in the same order."""
    import torch
    x, wg, wu = make(cuda, 3000, 1024, 512, seed=21)      # four hidden tiles: the wide pair form applies
    outs = []
    for rows, pair, wide in ((128, 0, 1), (256, 0, 1), (0, 1, 0), (0, 1, 1)):
        fpt.call("fpt_set_tuning", b"gate_up_tile_rows", rows)
        fpt.call("fpt_set_tuning", b"gate_up_cta_pair", pair)
        fpt.call("fpt_set_tuning", b"gate_up_pair_wide", wide)
        outs.append(gate_up(fpt, x, wg, wu))
    fpt.call("fpt_set_tuning", b"gate_up_tile_rows", 0)
    fpt.call("fpt_set_tuning", b"gate_up_cta_pair", -1)
    fpt.call("fpt_set_tuning", b"gate_up_pair_wide", 0)
    assert all(torch.equal(outs[0], other) for other in outs[1:])


def test_many_groups_like_routed_experts(fpt, cuda, tile_rows):
    """64 groups with Zipf-like sizes (some empty), the B4 layout at a size the check finishes quickly."""
    import torch
    rows, dim, hidden, groups = 9000, 512, 128, 64
    x, wg, wu = make(cuda, rows, dim, hidden, groups=groups, seed=11)
    weights = 1.0 / torch.arange(1, groups + 1, dtype=torch.float64) ** 1.1
    counts = torch.multinomial(weights / weights.sum(), rows, replacement=True,
                               generator=torch.Generator().manual_seed(5)).bincount(minlength=groups)
    counts[7] += counts[9]
    counts[9] = 0
    ends = torch.cumsum(counts, 0).to(torch.int32).to(cuda)
    raw = gate_up(fpt, x, wg, wu, ends, raw=True)
    want = products_fp32(x, wg, wu, ends)
    assert float((raw.float() - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())


def test_python_wrapper_and_adapters(cuda):
    import torch
    from torch import nn

    from fast_polynomial_transcendentals_b200.gate_up import gate_up_swiglu
    from fast_polynomial_transcendentals_b200.sfu_repro import adapters

    class Mlp(nn.Module):
        def __init__(self, dim, hidden):
            super().__init__()
            self.gate_proj, self.up_proj = nn.Linear(dim, hidden, bias=False), nn.Linear(dim, hidden, bias=False)
            self.down_proj = nn.Linear(hidden, dim, bias=False)
            self.act_fn = nn.SiLU()

        def forward(self, x):
            return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))

    torch.manual_seed(0)
    dim, hidden = 256, 384
    holder = nn.Sequential(Mlp(dim, hidden)).to(cuda, torch.bfloat16)
    x = torch.randn(3, 50, dim, device=cuda, dtype=torch.bfloat16)
    with torch.no_grad():
        exact = holder(x).float()
    assert adapters.fuse_gate_up_projections(holder, fuse_projection=True) == 1
    mlp = holder[0]
    with torch.no_grad():
        fused = mlp(x)                                     # one kernel for projection + activation
    mlp.sfu_fused_projection = None
    with torch.no_grad():
        two_step = mlp(x)                                  # cuBLAS projection, packed SwiGLU kernel
    scale = float(exact.abs().max())
    assert float((fused.float() - exact).abs().max()) < 5e-2 * scale
    assert float((fused.float() - two_step.float()).abs().max()) < 2e-2 * scale
    # with gradients recorded the module keeps the two-step path (the products are needed for the backward pass)
    mlp.sfu_fused_projection = {"degree": 3, "coeff_source": "current"}
    y = mlp(x.clone().requires_grad_(True))
    y.sum().backward()
    # "recompute": the fused kernel in training too; its backward recomputes the products.  Gradients against the two-step path.
    def grads(module):
        module.zero_grad(set_to_none=True)
        xin = x.clone().requires_grad_(True)
        (module(xin).float() * probe).sum().backward()
        return xin.grad.float(), module.w_in.weight.grad.float().clone()
    probe = torch.randn(3, 50, dim, device=cuda)
    mlp.sfu_fused_projection = None
    want_x, want_w = grads(mlp)
    mlp.sfu_fused_projection = {"degree": 3, "coeff_source": "current", "recompute": True}
    got_x, got_w = grads(mlp)
    assert float((got_x - want_x).abs().max()) < 2e-2 * float(want_x.abs().max())
    assert float((got_w - want_w).abs().max()) < 2e-2 * float(want_w.abs().max())
    compiled = torch.compile(lambda t: torch.ops.fpt_gate_up.swiglu(t, mlp.w_in.weight[:hidden], mlp.w_in.weight[hidden:], 3, 0),
                             fullgraph=True)
    with torch.no_grad():
        assert torch.equal(compiled(x), gate_up_swiglu(x, mlp.w_in.weight[:hidden], mlp.w_in.weight[hidden:]))
    # wrapper checks come before any launch
    w = mlp.w_in.weight
    with pytest.raises(RuntimeError):
        gate_up_swiglu(x.float(), w[:hidden], w[hidden:])
    with pytest.raises(RuntimeError):
        gate_up_swiglu(x, w[:hidden], w[hidden:hidden + 128])
    with pytest.raises(RuntimeError):
        gate_up_swiglu(x[..., :128], w[:hidden], w[hidden:])
    raw = gate_up_swiglu(x, w[:hidden], w[hidden:], raw=True)
    assert raw.shape == (3, 50, 2 * hidden)


def test_grouped_adapter_matches_the_three_product_path(cuda):
    import torch

    from fast_polynomial_transcendentals_b200.sfu_repro import adapters
    if not hasattr(torch, "_grouped_mm"):
        pytest.skip("torch._grouped_mm is not available")
    torch.manual_seed(1)
    experts, dim, hidden, rows = 8, 256, 128, 1024
    w1 = (torch.randn(experts, hidden, dim, device=cuda) * dim ** -0.5).to(torch.bfloat16)
    w3 = (torch.randn(experts, hidden, dim, device=cuda) * dim ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(experts, dim, hidden, device=cuda) * hidden ** -0.5).to(torch.bfloat16)
    x = torch.randn(rows, dim, device=cuda, dtype=torch.bfloat16)
    counts = torch.tensor([100, 0, 300, 24, 200, 150, 250, 0], device=cuda)
    from fast_polynomial_transcendentals_b200.sfu_repro.activations import resolve_mlp_activation_mul_impl
    _, activation_mul = resolve_mlp_activation_mul_impl("spline_silu_compile", degree=3, coeff_source="current")
    with torch.no_grad():
        two_step = adapters.run_grouped_experts(w1, w2, w3, x, counts, activation_mul)
        fused = adapters.run_grouped_experts(w1, w2, w3, x, counts, activation_mul, {"degree": 3, "coeff_source": "current"})
    assert float((fused[:1024].float() - two_step[:1024].float()).abs().max()) < 2e-2 * float(two_step.float().abs().max())


def test_random_shapes_every_form(fpt, cuda):
    """Eighty seeded random problems (1..200 groups with empty and ragged ones, rows the groups do not cover, K blocks that
    end inside a tile, tiny and odd sizes) through every form of the kernel: products against an fp32 product per group,
    nothing written outside the groups, no status word."""
    import random

    import torch
    rng = random.Random(20240611)
    for _ in range(80):
        groups = rng.choice([1, 1, 2, 3, 7, 16, 64, 200])
        rows = rng.choice([1, 5, 127, 128, 129, 255, 256, 257, 300, 1000, 2049, rng.randint(1, 6000)])
        dim = rng.choice([8, 64, 72, 128, 200, 512])
        hidden = 128 * rng.choice([1, 1, 2, 3, 4])
        form = rng.choice([(0, -1), (128, 0), (256, 0), (0, 1), (0, 0)])
        wide = rng.choice([0, 1])
        x, wg, wu = make(cuda, rows, dim, hidden, groups=max(groups, 2), seed=rows + dim)
        wg, wu = wg[:groups].contiguous(), wu[:groups].contiguous()
        last = rng.choice([rows, rows, max(0, rows - rng.randint(0, 300))])
        cuts = sorted(rng.randint(0, last) for _ in range(groups - 1)) + [last]
        ends = torch.tensor(cuts, dtype=torch.int32, device=cuda)
        fpt.call("fpt_set_tuning", b"gate_up_tile_rows", form[0])
        fpt.call("fpt_set_tuning", b"gate_up_cta_pair", form[1])
        fpt.call("fpt_set_tuning", b"gate_up_pair_wide", wide)
        try:
            raw = gate_up(fpt, x, wg, wu, ends, raw=True, fill=7.0)
            fused = gate_up(fpt, x, wg, wu, ends, fill=7.0)
        finally:
            fpt.call("fpt_set_tuning", b"gate_up_tile_rows", 0)
            fpt.call("fpt_set_tuning", b"gate_up_cta_pair", -1)
            fpt.call("fpt_set_tuning", b"gate_up_pair_wide", 0)
        what = (groups, rows, dim, hidden, form, wide, last)
        assert bool((raw[last:] == 7.0).all()) and bool((fused[last:] == 7.0).all()), what
        if last:
            want = products_fp32(x, wg, wu, ends)[:last]
            assert float((raw[:last].float() - want).abs().max()) <= 2.0 ** -7 * max(float(want.abs().max()), 1e-3) + 1e-6, what
            assert not bool(torch.isnan(fused[:last].float()).any()), what


def test_raw_epilogue_is_a_plain_grouped_product(cuda):
    """`grouped_linear`: one weight seen as two halves of output columns; against an fp32 product per group, dense and grouped."""
    import torch

    from fast_polynomial_transcendentals_b200.gate_up import grouped_linear
    torch.manual_seed(3)
    rows, dim, out_dim, groups = 1500, 1408, 512, 5
    x = torch.randn(rows, dim, device=cuda).to(torch.bfloat16)
    w = (torch.randn(groups, out_dim, dim, device=cuda) * dim ** -0.5).to(torch.bfloat16)
    ends = torch.tensor([100, 100, 700, 1400, 1500], dtype=torch.int32, device=cuda)
    got = grouped_linear(x, w, group_ends=ends).float()
    begin = 0
    for gi, end in enumerate(ends.tolist()):
        want = x[begin:end].float() @ w[gi].float().T
        if end > begin:
            assert float((got[begin:end] - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())
        begin = end
    dense = grouped_linear(x, w[0]).float()
    want = x.float() @ w[0].float().T
    assert float((dense - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())
    with pytest.raises(RuntimeError):
        grouped_linear(x, w[0, :384])


def test_argument_errors_come_back_as_status_codes(fpt, cuda):
    import torch
    x, wg, wu = make(cuda, 128, 64, 128)
    out = torch.empty(128, 128, dtype=torch.bfloat16, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    lib = fpt.load()

    def rc(**kw):
        a = dict(out=out.data_ptr(), x=x.data_ptr(), wg=wg.data_ptr(), wu=wu.data_ptr(), rows=128, dim=64, hidden=128, x_ld=64,
                 w_ld=64, w_gs=0, out_ld=128, ends=None, groups=1, degree=3, source=0, epilogue=0, status=status.data_ptr())
        a.update(kw)
        return lib.fpt_gate_up_swiglu(a["out"], a["x"], a["wg"], a["wu"], a["rows"], a["dim"], a["hidden"], a["x_ld"], a["w_ld"],
                                      a["w_gs"], a["out_ld"], a["ends"], a["groups"], a["degree"], a["source"], a["epilogue"],
                                      a["status"], stream())
    assert rc() == 0
    assert rc(hidden=96) != 0 and rc(dim=60) != 0            # unsupported shapes
    assert rc(status=None) != 0 and rc(out=None) != 0        # null pointers
    assert rc(groups=2) != 0                                 # several groups need their ends
    assert rc(groups=300) != 0
    assert rc(degree=4) != 0                                 # only the cubic (and degree 0) in the epilogue
    assert rc(epilogue=5) != 0
    assert rc(out_ld=64) != 0 and rc(x_ld=32) != 0
    assert rc(out=out.data_ptr() + 2) != 0                   # misaligned output
    assert rc(rows=0) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
