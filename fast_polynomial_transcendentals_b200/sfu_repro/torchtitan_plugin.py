"""The B1-B5 model converter for a TorchTitan-style trainer, on this package's kernels.

Mirrors the converter the reference registers with TorchTitan (reference: src/sfu_repro/torchtitan/plugin.py:386-482
`SFUReproConverter`, :362-383 case -> attention configuration, :197-265 fused gate/up MLP, :313-372 routed experts): same
class name, constructor checks, error messages and `convert(model)` contract -- one intervention per job, selected by
`job_config.sfu.case` in {b1..b5} and `job_config.sfu.variant`:

    b1   every SiLU-gated MLP -> one [dim -> 2 hidden] projection + packed SwiGLU (`adapters.fuse_gate_up_projections`)
    b2   attention -> tanh soft-cap, native (SFU) or polynomial           (`fa4.b2_component_configs`)
    b3   attention -> sigmoid attention, SFU or the direct D3 / D4 pair   (`fa4.b3_component_configs`, 4096 keys)
    b4   routed experts -> grouped GEMMs with the fused SwiGLU between    (`adapters.patch_grouped_experts`)
    b5   attention -> soft-max with routed software exponentials          (`fa4.b5_component_configs`)

TorchTitan itself is not a dependency: modules qualify by structure (`inner_attention` + `head_dim`; gate / up / down or
w1 / w3 / w2 projections; three-dimensional expert weights), so the converter also serves a model that merely looks like
TorchTitan's.  `register()` hands the class to TorchTitan's registry under the reference's name when TorchTitan can be
imported, and says so when it cannot.  The reference's dataset and model-spec registrations (training plumbing) are not
mirrored.
"""
from __future__ import annotations

import logging
from typing import Any

from torch import nn

from . import adapters
from .fa4 import (FA4Config, b2_component_configs, b3_component_configs, b5_component_configs, patch_attention_modules,
                  resolve_fa4_config)

LOGGER = logging.getLogger(__name__)
CONVERTER_NAME = "sfu_repro"


def attention_config(case: str, variant: str) -> FA4Config | None:
    """The attention configuration a case installs (none for b4; b1 keeps the plain soft-max)."""
    if case == "b1":
        return FA4Config(mode="softmax")
    if case == "b2":
        return b2_component_configs()[variant]
    if case == "b3":
        return b3_component_configs(sequence_length=4096)[variant]
    if case == "b5":
        return b5_component_configs()[variant]
    return None


def _reset_inserted_norms(model: nn.Module) -> int:
    """Give every patched attention module an `init_weights` that also resets the q / k norms the sigmoid wrapper adds
    (the reference swaps the module's class for that; here the bound method is wrapped)."""
    patched = 0
    for module in model.modules():
        inner = getattr(module, "inner_attention", None)
        if inner is None or not hasattr(inner, "config"):
            continue
        original = getattr(module, "init_weights", None)
        if original is not None and not getattr(original, "_sfu_wrapped", False):
            def init_weights(*args, _original=original, _inner=inner, **kwargs):
                result = _original(*args, **kwargs)
                for norm in (getattr(_inner, "q_norm", None), getattr(_inner, "k_norm", None)):
                    if norm is not None:
                        norm.reset_parameters()
                return result
            init_weights._sfu_wrapped = True
            module.init_weights = init_weights
        patched += 1
    return patched


class SFUReproConverter:
    """Apply one B1-B5 intervention to a model; `job_config` carries `.sfu.{case, variant, strict}`, `.model.name`,
    `.training.{seq_len, local_batch_size, global_batch_size, steps}` and `.compile.enable`; `parallel_dims` carries `.tp`."""

    def __init__(self, job_config: Any, parallel_dims: Any):
        self.job_config = job_config
        self.parallel_dims = parallel_dims
        self.case = str(job_config.sfu.case).lower()
        self.variant = str(job_config.sfu.variant).lower()
        self.strict = bool(job_config.sfu.strict)
        if self.case not in {"b1", "b2", "b3", "b4", "b5"}:
            raise ValueError(f"unknown SFU case {self.case!r}")
        allowed = set(b5_component_configs()) if self.case == "b5" else {"native", "polynomial"}
        if self.variant not in allowed:
            raise ValueError(f"unknown SFU variant {self.variant!r}")
        expected_model = "sfu_deepseek_v3" if self.case == "b4" else "sfu_llama3"
        if self.strict and job_config.model.name != expected_model:
            raise ValueError(f"{self.case.upper()} requires model.name={expected_model!r}, got {job_config.model.name!r}")
        if self.case == "b3" and int(job_config.training.seq_len) != 4096:
            raise ValueError("B3's direct D3/D4 fit requires training.seq_len=4096")
        if self.case == "b5" and int(job_config.training.seq_len) != 4096:
            raise ValueError("B5's routed-exp2 probe requires training.seq_len=4096")
        if self.case == "b5" and bool(job_config.compile.enable):
            raise ValueError("B5's public model probe requires compile.enable=false")
        if self.case == "b5" and self.strict:
            shape = (int(job_config.training.local_batch_size), int(job_config.training.global_batch_size),
                     int(job_config.training.steps))
            if shape != (1, 1, 80):
                raise ValueError(f"B5's public model probe requires local/global batch 1 and 80 steps, got {shape}")
        if self.case == "b1" and parallel_dims.tp != 1:
            raise ValueError("B1's fused gate/up projection requires tensor_parallel_degree=1")

    def convert(self, model: nn.Module) -> None:
        patched_attention = patched_activation = 0
        config = attention_config(self.case, self.variant)
        if config is not None:
            other = sorted({str(getattr(m, "attn_type", "unknown")) for m in model.modules()
                            if hasattr(m, "inner_attention") and hasattr(m, "attn_type") and m.attn_type != "sdpa"})
            if other:
                raise ValueError(f"{self.case.upper()} requires TorchTitan SDPA attention before the FA4 adapter; observed {other}")
            resolved = resolve_fa4_config(config, sequence_length=int(self.job_config.training.seq_len))
            patched_attention = patch_attention_modules(model, resolved)
            initialised = _reset_inserted_norms(model)
            if initialised != patched_attention:
                raise RuntimeError(f"FA4 patch count and initialization-hook count disagree: {patched_attention} != {initialised}")
        # not in the reference: `job_config.sfu.fuse_projection` (False / True / "recompute") also puts the SwiGLU into the
        # epilogue of the input projection(s) where the pass allows it (see adapters.fuse_gate_up_projections)
        fuse_projection = getattr(self.job_config.sfu, "fuse_projection", False)
        if self.case == "b1":
            patched_activation = adapters.fuse_gate_up_projections(model, variant=self.variant, degree=3,
                                                                   coeff_source="current", backward_impl="matched",
                                                                   fuse_projection=fuse_projection)
        elif self.case == "b4":
            patched_activation = adapters.patch_grouped_experts(model, variant=self.variant, degree=3, coeff_source="current",
                                                                fuse_projection=bool(fuse_projection))
        expected = 29 if self.case == "b4" else int(getattr(model, "n_layers", 0))
        observed = patched_activation if self.case in {"b1", "b4"} else patched_attention
        if self.strict and observed != expected:
            raise RuntimeError(f"{self.case.upper()} {self.variant} expected {expected} patched modules, observed {observed}")
        LOGGER.info("Configured %s %s: attention modules=%d, activation modules=%d", self.case.upper(), self.variant,
                    patched_attention, patched_activation)

    def post_optimizer_hook(self, model: nn.Module | list[nn.Module]) -> None:
        del model


def register() -> bool:
    """Register the converter with TorchTitan under the reference's name; False (and a log line) where TorchTitan is not
    installed.  Nothing else in this module needs TorchTitan."""
    try:
        from torchtitan.protocols import model_converter
    except ImportError:
        LOGGER.info("TorchTitan is not installed: SFUReproConverter is usable directly but not registered")
        return False
    registry = getattr(model_converter, "_registry_model_converter_cls", {})
    if registry.get(CONVERTER_NAME) is not SFUReproConverter:      # registering twice is an error in TorchTitan
        model_converter.register_model_converter(SFUReproConverter, CONVERTER_NAME)
    return True


__all__ = ["CONVERTER_NAME", "SFUReproConverter", "attention_config", "register"]
