"""Name -> callable resolution for MLP activations, on top of this package's kernels.

Mirrors the reference's resolver (reference: src/sfu_repro/activations.py:17-26 public names, :35-51 Sollya gate,
:119-136 fused-path check, :184-346 the three resolvers): the same activation names, labels, defaults and errors, the
same refusal of Sollya coefficients unless ``SFU_REPRO_ALLOW_SOLLYA_SWEEP`` is set, and the same guarantee that a
"current"-coefficient ``spline_silu_compile`` request really lands on the fused dispatcher operator.
"""
from __future__ import annotations

import os
from functools import lru_cache
from typing import Any

import torch
import torch.nn.functional as F

PUBLIC_MLP_ACTIVATIONS = ("native_silu", "spline_silu", "spline_silu_compile", "native_gelu", "spline_gelu",
                          "spline_gelu_compile")
_COEFF_SOURCE_TO_ID = {"current": 0, "sollya": 1}


def _env_flag(name: str) -> bool:
    value = os.environ.get(name)
    return value is not None and value.lower() in ("1", "true", "yes", "on")


def _ensure_coeff_source_allowed(coeff_source: str) -> None:
    if coeff_source not in _COEFF_SOURCE_TO_ID:
        raise ValueError(f"unknown coeff_source {coeff_source!r}; expected one of {tuple(_COEFF_SOURCE_TO_ID)}")
    if coeff_source == "sollya" and not _env_flag("SFU_REPRO_ALLOW_SOLLYA_SWEEP"):
        raise ValueError("Sollya coefficients are benchmark-only. Set SFU_REPRO_ALLOW_SOLLYA_SWEEP=1 for an explicit sweep.")


def _coeff_source_id(coeff_source: str) -> int:
    _ensure_coeff_source_allowed(coeff_source)
    return _COEFF_SOURCE_TO_ID[coeff_source]


@lru_cache(maxsize=1)
def load_spline_ops():
    """The operator module; raises RuntimeError when the CUDA library has not been built (no fallback exists)."""
    try:
        from .. import spline_ops
        from .. import _lib
        _lib.load()
    except (ImportError, OSError) as error:
        raise RuntimeError("The compiled kernel library is unavailable. Build it with "
                           "`python -m fast_polynomial_transcendentals_b200.build` first.") from error
    return spline_ops


@lru_cache(maxsize=1)
def _spline_compile():
    try:
        from .. import spline_compile
    except (ImportError, OSError) as error:
        raise RuntimeError("spline_compile is unavailable. Build the kernel library first.") from error
    return spline_compile


def _contiguous(tensor: torch.Tensor) -> torch.Tensor:
    return tensor if tensor.is_contiguous() else tensor.contiguous()


def _require_fused_current_swiglu(name: str, coeff_source: str, function: Any, role: str, expected_op: str) -> None:
    if name != "spline_silu_compile" or coeff_source != "current":
        return
    resolved_op = getattr(function, "__spline_op__", None)
    if resolved_op != expected_op:
        callable_name = getattr(function, "__name__", "")
        raise RuntimeError(
            f"{role} requested the production fused path but resolved to {callable_name or function!r} "
            f"({resolved_op=!r}) instead of {expected_op!r}. Check SPLINE_COMPILE_DISABLE_FUSED_SWIGLU and "
            "rebuild spline_ops.")


def _direct(kind: str, degree: int, coeff_source: str):
    """Direct (non-dispatcher) callables: the autograd entry when a gradient is wanted, the plain kernel otherwise."""
    ops = load_spline_ops()
    source_id = _coeff_source_id(coeff_source)
    plain = {"silu": ops.swish_fwd_variant, "gelu": ops.gelu_fwd_variant}[kind]
    with_grad = {"silu": ops.swish_ag_variant, "gelu": ops.gelu_ag_variant}[kind]

    def activation(tensor: torch.Tensor) -> torch.Tensor:
        tensor = _contiguous(tensor)
        if torch.is_grad_enabled() and tensor.requires_grad:
            return with_grad(tensor, degree, source_id)
        return plain(tensor, degree, source_id)

    activation.__name__ = f"spline_{kind}_d{degree}_{coeff_source}_direct"
    return activation


def _direct_silu_mul(degree: int, coeff_source: str):
    ops = load_spline_ops()
    source_id = _coeff_source_id(coeff_source)
    if source_id != 0:
        return None

    def activation_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        gate, up = _contiguous(gate), _contiguous(up)
        if torch.is_grad_enabled() and (gate.requires_grad or up.requires_grad):
            return ops.swish_mul_ag_variant(gate, up, degree, source_id)
        return ops.swish_mul_fwd_variant(gate, up, degree, source_id)

    activation_mul.__name__ = f"spline_silu_mul_d{degree}_{coeff_source}_direct"
    return activation_mul


def resolve_mlp_activation_impl(name: str, *, degree: int | None = None, coeff_source: str = "current"):
    """(label, callable) for an element-wise activation."""
    if name == "native_silu":
        return "native_silu", F.silu
    if name == "native_gelu":
        return "native_gelu", F.gelu
    if name in ("spline_silu", "spline_gelu"):
        kind = name.split("_")[1]
        resolved = (3 if kind == "silu" else 5) if degree is None else int(degree)
        return f"{name}[d{resolved},{coeff_source}]", _direct(kind, resolved, coeff_source)
    if name in ("spline_silu_compile", "spline_gelu_compile"):
        _ensure_coeff_source_allowed(coeff_source)
        sc = _spline_compile()
        kind = name.split("_")[1]
        resolved = (3 if kind == "silu" else 5) if degree is None else int(degree)
        default, factory = (sc.spline_silu, sc.make_spline_silu) if kind == "silu" else (sc.spline_gelu, sc.make_spline_gelu)
        activation = default if degree is None and coeff_source == "current" else factory(degree=resolved, coeff_source=coeff_source)
        return f"{name}[d{resolved},{coeff_source}]", activation
    raise ValueError(f"unknown activation {name!r}; expected one of " + ", ".join(PUBLIC_MLP_ACTIVATIONS))


def resolve_mlp_activation_mul_impl(name: str, *, degree: int | None = None, coeff_source: str = "current"):
    """(label, callable) for ``activation(gate) * up``; the fused kernel wherever one exists."""
    if name == "native_silu":
        return "native_silu_mul", lambda gate, up: F.silu(gate) * up
    if name == "spline_silu":
        resolved = 3 if degree is None else int(degree)
        activation_mul = _direct_silu_mul(resolved, coeff_source)
        if activation_mul is not None:
            return f"spline_silu_mul[d{resolved},{coeff_source}]", activation_mul
    if name == "spline_silu_compile":
        _ensure_coeff_source_allowed(coeff_source)
        resolved = 3 if degree is None else int(degree)
        activation_mul = _spline_compile().make_spline_silu_mul(degree=resolved, coeff_source=coeff_source)
        _require_fused_current_swiglu(name, coeff_source, activation_mul, "SwiGLU activation-multiply",
                                      "spline_ops::swish_mul_variant_fwd")
        implementation = ("spline_ops::swish_mul_variant_fwd" if coeff_source == "current"
                          else "spline_silu_compile_mul_unfused")
        return f"{implementation}[d{resolved},{coeff_source}]", activation_mul
    activation_name, activation = resolve_mlp_activation_impl(name, degree=degree, coeff_source=coeff_source)
    return f"{activation_name}_mul", lambda gate, up: activation(gate) * up


def resolve_mlp_activation_packed_impl(name: str, *, degree: int | None = None, coeff_source: str = "current",
                                       backward_impl: str = "matched"):
    """(label, callable) for a packed ``[..., 2 * hidden]`` SwiGLU."""
    if backward_impl not in ("matched", "native"):
        raise ValueError("backward_impl must be 'matched' or 'native'")
    if name == "native_silu":
        return "native_silu_packed", _spline_compile().make_native_silu_packed()
    if name == "spline_silu_compile":
        _ensure_coeff_source_allowed(coeff_source)
        resolved = 3 if degree is None else int(degree)
        activation = _spline_compile().make_spline_silu_packed(degree=resolved, coeff_source=coeff_source,
                                                               backward_impl=backward_impl)
        expected_op = ("spline_ops::swish_mul_packed_variant_fwd" if backward_impl == "matched"
                       else "spline_ops::swish_mul_packed_native_bwd_fwd")
        _require_fused_current_swiglu(name, coeff_source, activation, "packed SwiGLU", expected_op)
        return f"{expected_op}[d{resolved},{coeff_source},{backward_impl}_bwd]", activation
    activation_name, activation_mul = resolve_mlp_activation_mul_impl(name, degree=degree, coeff_source=coeff_source)

    def activation_packed(packed: torch.Tensor) -> torch.Tensor:
        gate, up = packed.chunk(2, dim=-1)
        return activation_mul(gate, up)

    return f"{activation_name}_packed", activation_packed


__all__ = ["PUBLIC_MLP_ACTIVATIONS", "load_spline_ops", "resolve_mlp_activation_impl",
           "resolve_mlp_activation_mul_impl", "resolve_mlp_activation_packed_impl"]
