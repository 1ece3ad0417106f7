"""CPU: the configuration / patching layer (sfu_repro.fa4, sfu_repro.activations, rope evaluator, spline_compile fakes)."""
import math
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

from fast_polynomial_transcendentals_b200 import spline_compile
from fast_polynomial_transcendentals_b200.sfu_repro import activations, fa4
from fast_polynomial_transcendentals_b200.sfu_repro.rope import (SOLLYA_D3_D4, UNIFORM_D5_D4, UNIFORM_D7_D6, polynomial_sincos,
                                                                 reduce_to_quarter_turn, rope_phase_increments)

ROOT = Path(__file__).resolve().parents[1]
REFERENCE_TEST = Path(os.environ.get("FPT_REFERENCE_ROOT", ROOT.parent / "reference")) / "tests" / "test_fa4_config.py"


def test_canonical_attention_configs_resolve_against_our_runtime():
    b2 = fa4.resolve_fa4_config(fa4.b2_component_configs()["polynomial"])
    assert b2.mode == "softcap" and b2.softcap == 0.0 and b2.score_mod == fa4.SoftcapScoreMod(30.0, 4, "device", "current")
    b3 = fa4.resolve_fa4_config(fa4.b3_component_configs()["polynomial"], sequence_length=4096)
    assert b3.sigmoid_attention and b3.sigmoid_sfu_res == 0 and b3.sigmoid_use_direct_bwd_poly and b3.sigmoid_degree_bwd == 4
    assert set(fa4.b5_component_configs()) == {"native", "pwl2_safe_f16", "d2_safe"}


@pytest.mark.parametrize("length", [1024, 4095, 8192, 16384])
def test_direct_sigmoid_rejects_every_length_but_4096(length):
    with pytest.raises(ValueError, match="4096"):
        fa4.b3_component_configs(sequence_length=length)
    with pytest.raises(ValueError, match="fitted for sequence length 4096"):
        fa4.validate_fa4_config(fa4.b3_component_configs()["polynomial"], sequence_length=length)


def test_exp2_variant_parsing_and_validation():
    variants = fa4.parse_exp2_variants(fa4.DEFAULT_EXP2_VARIANTS)
    assert variants[0].name == "sfu" and variants[1].forward_frequency is None
    assert variants[-1].nominal_forward_polynomial_fraction == 1.0
    for bad in ("x=d3:3:0", "x=d3:5:0", "x=nope:0:0", "=d3:0:0", "x=d3:0", "a=d3:0:0,a=d3:4:0"):
        with pytest.raises(ValueError):
            fa4.parse_exp2_variants(bad)
    with pytest.raises(ValueError, match="native softcap requires"):
        fa4.validate_fa4_config(fa4.FA4Config(mode="softcap", softcap_backend="native"))
    with pytest.raises(ValueError, match="Sollya"):
        fa4.validate_fa4_config(fa4.FA4Config(mode="softcap", softcap_backend="device", softcap_coeff_source="sollya"))


def test_the_reference_s_own_config_tests_pass_against_this_module():
    """Where a reference checkout is mounted, its test file is run unchanged with `sfu_repro` aliased to this package."""
    if not REFERENCE_TEST.exists():
        pytest.skip("no reference checkout here")
    code = textwrap.dedent(f"""
        import sys, pytest
        sys.path.insert(0, {str(ROOT)!r})
        import fast_polynomial_transcendentals_b200.sfu_repro.fa4
        for name in ("", ".fa4"):
            sys.modules["sfu_repro" + name] = sys.modules["fast_polynomial_transcendentals_b200.sfu_repro" + name]
        sys.exit(pytest.main(["-q", "-p", "no:cacheprovider", "--rootdir", "/tmp", {str(REFERENCE_TEST)!r}]))
    """)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]


def test_activation_names_labels_and_sollya_gate(monkeypatch):
    assert activations.resolve_mlp_activation_impl("native_silu")[0] == "native_silu"
    label, fn = activations.resolve_mlp_activation_impl("spline_silu_compile")
    assert label == "spline_silu_compile[d3,current]" and fn is spline_compile.spline_silu
    label, fn = activations.resolve_mlp_activation_mul_impl("spline_silu_compile", degree=3)
    assert label == "spline_ops::swish_mul_variant_fwd[d3,current]" and fn.__spline_op__ == "spline_ops::swish_mul_variant_fwd"
    label, fn = activations.resolve_mlp_activation_packed_impl("spline_silu_compile", degree=3, backward_impl="native")
    assert label == "spline_ops::swish_mul_packed_native_bwd_fwd[d3,current,native_bwd]"
    assert activations.resolve_mlp_activation_packed_impl("native_silu")[1].__spline_op__ == "spline_ops::swish_mul_packed_native_fwd"
    with pytest.raises(ValueError, match="benchmark-only"):
        activations.resolve_mlp_activation_impl("spline_silu_compile", coeff_source="sollya")
    with pytest.raises(ValueError, match="unknown activation"):
        activations.resolve_mlp_activation_impl("relu")
    monkeypatch.setenv("SFU_REPRO_ALLOW_SOLLYA_SWEEP", "1")
    assert activations.resolve_mlp_activation_mul_impl("spline_silu_compile", coeff_source="sollya")[0].startswith(
        "spline_silu_compile_mul_unfused")


def test_disabling_the_fused_path_is_detected(monkeypatch):
    monkeypatch.setenv("SPLINE_COMPILE_DISABLE_FUSED_SWIGLU", "1")
    spline_compile.make_spline_silu_mul.cache_clear()
    spline_compile.make_spline_silu_packed.cache_clear()
    try:
        with pytest.raises(RuntimeError, match="production fused path"):
            activations.resolve_mlp_activation_mul_impl("spline_silu_compile")
        with pytest.raises(RuntimeError, match="production fused path"):
            activations.resolve_mlp_activation_packed_impl("spline_silu_compile")
    finally:
        spline_compile.make_spline_silu_mul.cache_clear()
        spline_compile.make_spline_silu_packed.cache_clear()


def test_dispatcher_ops_have_shape_functions():
    x = torch.empty(6, 16, device="meta", dtype=torch.bfloat16)
    ops = torch.ops.spline_ops
    assert ops.swish_mul_packed_variant_fwd(x, 3, 0).shape == (6, 8)
    assert ops.swish_mul_variant_fwd(x, x, 3, 0).shape == x.shape
    gg, gu = ops.swish_mul_variant_bwd(x, x, x, 3, 0)
    assert gg.shape == gu.shape == x.shape
    assert ops.swish_mul_packed_variant_bwd(x[:, :8], x, 3, 0).shape == x.shape
    assert torch.ops.spline_compile.gelu_variant_fwd(x, 4, 0).shape == x.shape


def test_sincos_polynomial_budgets_and_quadrants():
    """Error budgets on 262145 points over +-131072 rad and the quadrant table (reference
    tests/test_rope_polynomial_sincos.py:91-135)."""
    a = torch.linspace(-131072, 131072, 262145, dtype=torch.float64)
    for poly, tol in ((SOLLYA_D3_D4, 2.1e-4), (UNIFORM_D5_D4, 4.5e-5), (UNIFORM_D7_D6, 1.2e-6)):
        c, s = polynomial_sincos(a, polynomial=poly)
        assert float((c.double() - torch.cos(a)).abs().max()) < tol
        assert float((s.double() - torch.sin(a)).abs().max()) < tol
    assert (SOLLYA_D3_D4.sin_degree, SOLLYA_D3_D4.cos_degree, UNIFORM_D7_D6.sin_degree) == (3, 4, 7)
    q = reduce_to_quarter_turn(torch.tensor([0, math.pi, 1.5 * math.pi, 2 * math.pi, 2.5 * math.pi, -math.pi]))[1]
    assert q.tolist() == [0, 2, 3, 0, 1, 2]
    with pytest.raises(TypeError):
        reduce_to_quarter_turn(torch.arange(4))
    inc = rope_phase_increments(128)
    assert inc.dtype == torch.int32 and inc.numel() == 64 and int(inc[0]) == 683565276


def test_every_name_of_the_reference_operator_module_exists():
    """The fixture lists what the reference's extension module and dispatcher library export
    (tests/golden/make_op_surface.py wrote it from the reference's C++ source)."""
    import json
    from pathlib import Path

    import torch

    from fast_polynomial_transcendentals_b200 import spline_compile, spline_ops  # noqa: F401  (registers the library)
    surface = json.loads((Path(__file__).parent / "golden" / "op_surface.json").read_text())
    missing = [name for name in surface["pybind"] if not callable(getattr(spline_ops, name, None))]
    assert not missing, missing
    missing = [name for name in surface["dispatcher"] if not hasattr(torch.ops.spline_ops, name)]
    assert not missing, missing


def test_module_surgery_finds_patches_and_restores_by_structure():
    """No kernel runs here: the adapters recognise gated MLPs, experts and activation slots by their attributes."""
    import torch
    from torch import nn

    from fast_polynomial_transcendentals_b200.sfu_repro import adapters

    class HF(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = nn.Linear(8, 16, bias=False), nn.Linear(8, 16, bias=False), nn.Linear(16, 8, bias=False)
            self.act_fn = nn.SiLU()

        def forward(self, x):
            return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))

    class Titan(nn.Module):
        def __init__(self):
            super().__init__()
            self.w1, self.w2, self.w3 = nn.Linear(8, 16, bias=False), nn.Linear(16, 8, bias=False), nn.Linear(8, 16, bias=False)

        def forward(self, x):
            return self.w2(torch.nn.functional.silu(self.w1(x)) * self.w3(x))

    class Experts(nn.Module):
        def __init__(self):
            super().__init__()
            self.w1, self.w2, self.w3 = (nn.Parameter(torch.zeros(2, 16, 8)), nn.Parameter(torch.zeros(2, 8, 16)),
                                         nn.Parameter(torch.zeros(2, 16, 8)))

        def forward(self, x, counts):
            return x

    model = nn.ModuleDict({"a": HF(), "b": Titan(), "c": Experts(), "d": nn.Linear(8, 8)})
    assert len(adapters.dense_swiglu_modules(model)) == 2
    x = torch.randn(3, 8)
    want = model["a"](x)
    assert adapters.patch_dense_swiglu(model) == 2
    assert adapters.patch_grouped_experts(model) == 1
    assert adapters.patch_activation_slots(model, kind="silu") == 1
    assert isinstance(model["a"].act_fn, adapters.FunctionActivation)
    assert adapters.restore(model) == 4
    assert isinstance(model["a"].act_fn, nn.SiLU) and "forward" not in model["a"].__dict__
    assert torch.equal(model["a"](x), want)
    before = sum(p.numel() for p in model.parameters())
    w1, w3 = model["b"].w1.weight.clone(), model["b"].w3.weight.clone()
    assert adapters.fuse_gate_up_projections(model) == 2
    assert sum(p.numel() for p in model.parameters()) == before
    assert torch.equal(model["b"].w_in.weight, torch.cat((w1, w3), dim=0))
    assert getattr(model["b"].sfu_activation_packed, "__spline_op__", None) == "spline_ops::swish_mul_packed_variant_fwd"


def test_gated_mlps_with_another_activation_are_not_turned_into_swiglu():
    """GeGLU / ReGLU MLPs have the same three projections as SwiGLU; patching them would silently change the model's
    function.  Only SiLU-gated modules qualify (the reference's own test, scripts/benchmark_open_weights.py:649-664)."""
    from torch import nn

    from fast_polynomial_transcendentals_b200.sfu_repro import adapters

    class Gated(nn.Module):
        def __init__(self, act, bias=False, names=("gate_proj", "up_proj", "down_proj")):
            super().__init__()
            for n, (i, o) in zip(names, ((16, 32), (16, 32), (32, 16))):
                setattr(self, n, nn.Linear(i, o, bias=bias))
            if act is not None:
                self.act_fn = act

    class Config:
        hidden_act = "silu"

    model = nn.ModuleDict({"silu": Gated(nn.SiLU()), "gelu": Gated(nn.GELU(approximate="tanh")), "relu": Gated(nn.ReLU()),
                           "functional": Gated(torch.nn.functional.silu), "slotless": Gated(None, names=("w1", "w3", "w2")),
                           "slotless_biased": Gated(None, bias=True)})
    model["by_config"] = Gated(nn.Identity())
    model["by_config"].config = Config()
    assert {n: adapters.gated_mlp_activation(m) == "silu" for n, m in model.items()} == {
        "silu": True, "gelu": False, "relu": False, "functional": True, "slotless": True, "slotless_biased": False,
        "by_config": True}
    skipped = []
    assert adapters.patch_dense_swiglu(model, skipped=skipped) == 4
    assert sorted(n for n, _ in skipped) == ["gelu", "relu", "slotless_biased"]
    assert "forward" not in model["gelu"].__dict__ and "forward" in model["silu"].__dict__
    assert adapters.restore(model) == 4
    skipped = []
    assert adapters.fuse_gate_up_projections(model, skipped=skipped) == 4
    assert isinstance(model["gelu"], Gated) and isinstance(model["relu"], Gated)
    assert isinstance(model["silu"], adapters.FusedGateUpFeedForward)
    assert sorted(n for n, _ in skipped) == ["gelu", "relu", "slotless_biased"]
