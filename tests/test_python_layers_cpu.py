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


def test_trainer_converter_checks_and_converts_by_structure():
    """The B1-B5 converter (reference: src/sfu_repro/torchtitan/plugin.py:386-482): constructor checks and messages, and
    `convert` on stand-in modules that only look like a trainer's (no trainer installed here)."""
    from types import SimpleNamespace as NS

    from torch import nn

    from fast_polynomial_transcendentals_b200.sfu_repro import adapters, torchtitan_plugin as plugin

    def job(case, variant="polynomial", strict=False, model="sfu_llama3", seq_len=4096, compile_enable=False,
            local=1, global_=1, steps=80):
        return NS(sfu=NS(case=case, variant=variant, strict=strict), model=NS(name=model), compile=NS(enable=compile_enable),
                  training=NS(seq_len=seq_len, local_batch_size=local, global_batch_size=global_, steps=steps))

    dims = NS(tp=1)
    for bad, message in ((job("b9"), "unknown SFU case"), (job("b2", "fast"), "unknown SFU variant"),
                         (job("b4", strict=True), "requires model.name='sfu_deepseek_v3'"),
                         (job("b3", seq_len=8192), "requires training.seq_len=4096"),
                         (job("b5", "d2_safe", compile_enable=True), "compile.enable=false"),
                         (job("b5", "d2_safe", strict=True, steps=10), "80 steps")):
        with pytest.raises(ValueError, match=message):
            plugin.SFUReproConverter(bad, dims)
    with pytest.raises(ValueError, match="tensor_parallel_degree=1"):
        plugin.SFUReproConverter(job("b1"), NS(tp=2))
    assert plugin.attention_config("b4", "polynomial") is None
    assert plugin.attention_config("b5", "pwl2_safe_f16").exp2_emu_freq_bwd == 32

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.head_dim, self.attn_type = 128, "sdpa"
            self.inner_attention = nn.Identity()
            self.wq = nn.Linear(8, 8)
            self.resets = 0

        def init_weights(self, init_std):
            self.resets += 1

    class FeedForward(nn.Module):
        def __init__(self):
            super().__init__()
            self.w1, self.w2, self.w3 = nn.Linear(16, 32, bias=False), nn.Linear(32, 16, bias=False), nn.Linear(16, 32, bias=False)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.attention, self.feed_forward = Attention(), FeedForward()

    class Model(nn.Module):
        def __init__(self, layers=3):
            super().__init__()
            self.n_layers = layers
            self.layers = nn.ModuleList(Block() for _ in range(layers))

    model = Model()
    plugin.SFUReproConverter(job("b1", strict=True), dims).convert(model)
    assert all(isinstance(b.feed_forward, adapters.FusedGateUpFeedForward) for b in model.layers)
    assert all(isinstance(b.attention.inner_attention, fa4.FA4AttentionWrapper) for b in model.layers)
    model = Model()
    plugin.SFUReproConverter(job("b3", strict=True), dims).convert(model)
    wrapper = model.layers[0].attention.inner_attention
    assert wrapper.config.sigmoid_attention and wrapper.q_norm is not None
    with torch.no_grad():
        wrapper.q_norm.weight.fill_(3.0)
    model.layers[0].attention.init_weights(0.02)          # resets the norms the wrapper added, then the module's own
    assert model.layers[0].attention.resets == 1 and float(wrapper.q_norm.weight[0]) == 1.0
    with pytest.raises(RuntimeError, match="expected 5 patched modules, observed 3"):
        bigger = Model()
        bigger.n_layers = 5
        plugin.SFUReproConverter(job("b2", "native", strict=True), dims).convert(bigger)
    flex = Model()
    flex.layers[1].attention.attn_type = "flex"
    with pytest.raises(ValueError, match="requires TorchTitan SDPA attention"):
        plugin.SFUReproConverter(job("b2"), dims).convert(flex)
    try:
        from torchtitan.protocols import model_converter
    except ImportError:
        assert plugin.register() is False                  # no trainer here: says so, does not fail
        return
    assert plugin.register() is True and plugin.register() is True          # idempotent
    assert model_converter._registry_model_converter_cls[plugin.CONVERTER_NAME] is plugin.SFUReproConverter
    # a real TorchTitan Llama (whatever version is installed): B1 replaces every feed-forward by the fused form
    from torchtitan.models.llama3.model.args import TransformerModelArgs
    from torchtitan.models.llama3.model.model import Transformer
    args = TransformerModelArgs(dim=64, n_layers=2, n_heads=2, n_kv_heads=1, vocab_size=128, multiple_of=16, max_seq_len=64)
    with torch.device("meta"):
        titan = Transformer(args)
    plugin.SFUReproConverter(job("b1", strict=True), dims).convert(titan)
    blocks = list(titan.layers.values()) if hasattr(titan.layers, "values") else list(titan.layers)
    assert len(blocks) == 2 and all(isinstance(b.feed_forward, adapters.FusedGateUpFeedForward) for b in blocks)
    hidden = blocks[0].feed_forward.w_out.weight.shape[1]
    assert blocks[0].feed_forward.w_in.weight.shape == (2 * hidden, 64)
