"""Module surgery that puts the fused polynomial kernels into existing models, by structure rather than by class.

The reference patches TorchTitan's Llama feed-forward and grouped experts (reference: src/sfu_repro/torchtitan/plugin.py:197-265
fused gate/up projection + packed SwiGLU, :294-372 routed experts) and Hugging Face MLPs and activation slots (reference:
scripts/benchmark_open_weights.py:1072-1158).  Neither framework is a dependency here: a module qualifies by its
attributes (`gate_proj / up_proj / down_proj` or `w1 / w3 / w2`), so the same functions serve both families.

Every patch is reversible (`restore(model)`) except the weight-fusing one, which rewrites parameters in place as the
reference does.
"""
from __future__ import annotations

from types import MethodType
from typing import Any, Callable

import torch
from torch import nn

from ..gate_up import gate_up_swiglu, gate_up_swiglu_recompute, grouped_linear
from .activations import (resolve_mlp_activation_impl, resolve_mlp_activation_mul_impl,
                          resolve_mlp_activation_packed_impl)

_ORIGINAL = "_sfu_original_forward"
_SLOT = "_sfu_original_activation"


def _projection_names(module: nn.Module) -> tuple[str, str, str] | None:
    """(gate, up, down) attribute names of a gated MLP, or None."""
    for names in (("gate_proj", "up_proj", "down_proj"), ("w1", "w3", "w2")):
        if all(isinstance(getattr(module, n, None), nn.Linear) for n in names):
            return names
    return None


_ACTIVATION_SLOTS = ("act_fn", "activation_fn", "act")


def _is_silu(module: nn.Module, fn: Any) -> bool:
    """The test the reference applies before it treats a gated MLP as SwiGLU (reference:
    scripts/benchmark_open_weights.py:649-664): the module's config names SiLU / swish, or the activation object is one."""
    config = getattr(module, "config", None)
    for name in (getattr(config, "hidden_act", None), getattr(config, "hidden_activation", None)):
        if isinstance(name, str) and name.lower() in ("silu", "swish"):
            return True
    if isinstance(fn, nn.SiLU) or fn is torch.nn.functional.silu:
        return True
    names = (type(fn).__name__.lower(), str(getattr(fn, "__name__", "")).lower())
    return any(n in ("silu", "swish", "siluactivation") for n in names)


def gated_mlp_activation(module: nn.Module) -> str:
    """'silu' when the gated MLP computes down(silu(gate(x)) * up(x)), else a description of what it holds instead.

    A module with an activation slot (`act_fn`, `activation_fn`, `act`) qualifies only if that slot is SiLU: a GELU- or
    ReLU-gated MLP has the same three projections and must not be turned into SwiGLU.  A module without any slot
    qualifies when all three projections are bias-free (the Llama feed-forward that calls `F.silu` in its forward,
    reference: src/sfu_repro/torchtitan/plugin.py:197-265)."""
    slots = [(a, getattr(module, a)) for a in _ACTIVATION_SLOTS if getattr(module, a, None) is not None]
    if slots:
        for _, fn in slots:
            if isinstance(fn, FunctionActivation) or _is_silu(module, fn):
                return "silu"
        return f"{slots[0][0]}={type(slots[0][1]).__name__}"
    names = _projection_names(module)
    if names and all(getattr(module, n).bias is None for n in names):
        return "silu"
    return "no activation slot and biased projections"


def dense_swiglu_modules(model: nn.Module, skipped: list[tuple[str, str]] | None = None) -> list[nn.Module]:
    """Gated MLPs whose activation is SiLU; the others are appended to `skipped` as (module name, what they hold)."""
    found = []
    for name, module in model.named_modules():
        if _projection_names(module) is None:
            continue
        kind = gated_mlp_activation(module)
        if kind == "silu":
            found.append(module)
        elif skipped is not None:
            skipped.append((name, kind))
    return found


def patch_dense_swiglu(model: nn.Module, *, variant: str = "polynomial", degree: int = 3,
                       coeff_source: str = "current", skipped: list[tuple[str, str]] | None = None) -> int:
    """down(act(gate(x)) * up(x)) with the fused SwiGLU kernel between the projections; weights untouched.  Gated MLPs
    whose activation is not SiLU are left alone and reported through `skipped`."""
    implementation = "native_silu" if variant == "native" else "spline_silu_compile"
    _, activation_mul = resolve_mlp_activation_mul_impl(implementation, degree=degree, coeff_source=coeff_source)
    patched = 0
    for module in dense_swiglu_modules(model, skipped):
        gate, up, down = _projection_names(module)

        def forward(self, x, *args, _g=gate, _u=up, _d=down, **kwargs):
            return getattr(self, _d)(activation_mul(getattr(self, _g)(x), getattr(self, _u)(x)))

        if _ORIGINAL not in module.__dict__:
            module.__dict__[_ORIGINAL] = module.forward
        module.forward = MethodType(forward, module)
        patched += 1
    return patched


class FusedGateUpFeedForward(nn.Module):
    """One [dim -> 2*hidden] projection, packed SwiGLU, one [hidden -> dim] projection (the B1 layout)."""

    def __init__(self, w_in: nn.Linear, w_out: nn.Linear, activation_packed: Callable[[torch.Tensor], torch.Tensor],
                 fused_projection: dict | None = None):
        super().__init__()
        self.w_in, self.w_out = w_in, w_out
        self.sfu_activation_packed = activation_packed
        # {"degree": ..., "coeff_source": ...}: run projection and activation as one kernel where no gradient is wanted
        self.sfu_fused_projection = fused_projection

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        fused = self.sfu_fused_projection
        if fused is not None and _fusable(x, self.w_in.weight, self.w_out.weight.shape[-1], fused.get("recompute", False)):
            hidden = self.w_out.weight.shape[-1]
            weight = self.w_in.weight
            op = gate_up_swiglu_recompute if fused.get("recompute", False) else gate_up_swiglu
            return self.w_out(op(x, weight[:hidden], weight[hidden:], degree=fused["degree"], coeff_source=fused["coeff_source"]))
        return self.w_out(self.sfu_activation_packed(self.w_in(x)))

    def init_weights(self, init_std: float) -> None:
        hidden = self.w_out.weight.shape[-1]
        nn.init.trunc_normal_(self.w_in.weight, mean=0.0, std=0.02)
        with torch.no_grad():
            self.w_in.weight[hidden:].mul_(init_std / 0.02)
        nn.init.trunc_normal_(self.w_out.weight, mean=0.0, std=init_std)


def _fusable(x: torch.Tensor, weight: torch.Tensor, hidden: int, recompute: bool = False) -> bool:
    """The one-kernel projection + SwiGLU serves bf16 CUDA inputs when no gradient is recorded (a backward pass needs the
    two products, which that kernel never stores) or when the caller accepts their recomputation in the backward pass."""
    if not recompute and torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        return False
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and hidden % 128 == 0
            and weight.shape[-1] % 8 == 0)


@torch.no_grad()
def fuse_gate_up_projections(model: nn.Module, *, variant: str = "polynomial", degree: int = 3,
                             coeff_source: str = "current", backward_impl: str = "matched",
                             skipped: list[tuple[str, str]] | None = None, fuse_projection: bool | str = False) -> int:
    """Replace every bias-free SiLU-gated MLP by `FusedGateUpFeedForward` with w_in = cat(gate, up) (rows); gated MLPs
    with another activation are left alone and reported through `skipped`.  `fuse_projection=True` also lets forward
    passes without gradients run the projection and the activation as one kernel (`gate_up.gate_up_swiglu`);
    `fuse_projection="recompute"` uses that kernel in training too: the `[rows, 2 hidden]` products are not kept but
    recomputed in the backward pass (one more projection per layer and step for 2 x rows x hidden x 2 bytes less memory)."""
    implementation = "native_silu" if variant == "native" else "spline_silu_compile"
    _, activation_packed = resolve_mlp_activation_packed_impl(implementation, degree=degree, coeff_source=coeff_source,
                                                              backward_impl=backward_impl)
    replaced = 0
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            names = _projection_names(child)
            if names is None:
                continue
            kind = gated_mlp_activation(child)
            if kind != "silu":
                if skipped is not None:
                    skipped.append((child_name, kind))
                continue
            gate, up, down = (getattr(child, n) for n in names)
            if gate.bias is not None or up.bias is not None:
                continue
            hidden, dim = gate.weight.shape
            device, dtype = gate.weight.device, gate.weight.dtype
            w_in = nn.Linear(dim, 2 * hidden, bias=False, device=device, dtype=dtype)
            w_out = nn.Linear(hidden, dim, bias=down.bias is not None, device=device, dtype=dtype)
            if device.type != "meta":
                w_in.weight.copy_(torch.cat((gate.weight, up.weight), dim=0))
                w_out.weight.copy_(down.weight)
                if down.bias is not None:
                    w_out.bias.copy_(down.bias)
            fused = ({"degree": 0 if variant == "native" else degree, "coeff_source": coeff_source,
                      "recompute": fuse_projection == "recompute"} if fuse_projection else None)
            setattr(parent, child_name, FusedGateUpFeedForward(w_in, w_out, activation_packed, fused))
            replaced += 1
    return replaced


def _is_grouped_experts(module: nn.Module) -> bool:
    weights = [getattr(module, n, None) for n in ("w1", "w2", "w3")]
    return all(isinstance(w, (torch.Tensor, nn.Parameter)) and w.dim() == 3 for w in weights)


def run_grouped_experts(w1, w2, w3, x, num_tokens_per_expert, activation_mul, fused_projection: dict | None = None) -> torch.Tensor:
    """Expert-sorted rows through three grouped GEMMs with the fused SwiGLU between them (the B4 site); with
    `fused_projection` and no gradient wanted, the first two and the activation are one kernel."""
    offsets = torch.cumsum(num_tokens_per_expert, dim=0, dtype=torch.int32)
    xb = x.bfloat16()
    if (fused_projection is not None and w1.dtype == torch.bfloat16 and w3.dtype == torch.bfloat16 and w1.shape[0] <= 256
            and w1.stride() == w3.stride() and _fusable(xb, w1, w1.shape[-2])):
        hidden = gate_up_swiglu(xb, w1, w3, group_ends=offsets, degree=fused_projection["degree"],
                                coeff_source=fused_projection["coeff_source"])
        if w2.dtype == torch.bfloat16 and w2.shape[-2] % 256 == 0 and w2.shape[-1] % 8 == 0 and w2.stride(-1) == 1:
            # the projection back runs on the same kernel (its raw epilogue is a plain grouped product); rows that no group
            # owns are left unwritten
            return grouped_linear(hidden, w2, group_ends=offsets).type_as(x)
    else:
        gate = torch._grouped_mm(xb, w1.bfloat16().transpose(-2, -1), offs=offsets)
        up = torch._grouped_mm(xb, w3.bfloat16().transpose(-2, -1), offs=offsets)
        hidden = activation_mul(gate, up)
    return torch._grouped_mm(hidden, w2.bfloat16().transpose(-2, -1), offs=offsets).type_as(x)


def patch_grouped_experts(model: nn.Module, *, variant: str = "polynomial", degree: int = 3,
                          coeff_source: str = "current", fuse_projection: bool = False) -> int:
    """Modules holding 3-D `w1 / w2 / w3` ([experts, hidden, dim], [experts, dim, hidden], [experts, hidden, dim])
    and called as `forward(x, num_tokens_per_expert)`.  `fuse_projection=True`: forward passes without gradients run
    the two input projections and the activation as one kernel."""
    implementation = "native_silu" if variant == "native" else "spline_silu_compile"
    _, activation_mul = resolve_mlp_activation_mul_impl(implementation, degree=degree, coeff_source=coeff_source)
    patched = 0
    for module in model.modules():
        if not _is_grouped_experts(module):
            continue

        def forward(self, x, num_tokens_per_expert):
            return run_grouped_experts(self.w1, self.w2, self.w3, x, num_tokens_per_expert, self.sfu_activation_mul,
                                       self.sfu_fused_projection)

        module.sfu_activation_mul = activation_mul
        module.sfu_fused_projection = ({"degree": 0 if variant == "native" else degree, "coeff_source": coeff_source}
                                       if fuse_projection else None)
        if _ORIGINAL not in module.__dict__:
            module.__dict__[_ORIGINAL] = module.forward
        module.forward = MethodType(forward, module)
        patched += 1
    return patched


class FunctionActivation(nn.Module):
    """An activation function in a slot that used to hold a module."""

    def __init__(self, function: Callable[[torch.Tensor], torch.Tensor]):
        super().__init__()
        self.function = function

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.function(x if x.is_contiguous() else x.contiguous())


def patch_activation_slots(model: nn.Module, *, kind: str = "silu", degree: int | None = None,
                           coeff_source: str = "current", attributes: tuple[str, ...] = _ACTIVATION_SLOTS) -> int:
    """Swap SiLU (or GELU) activations held in the usual attribute slots for the polynomial kernel."""
    targets = {"silu": (nn.SiLU, torch.nn.functional.silu), "gelu": (nn.GELU, torch.nn.functional.gelu)}[kind]
    _, activation = resolve_mlp_activation_impl(f"spline_{kind}_compile", degree=degree, coeff_source=coeff_source)
    patched = 0
    for module in model.modules():
        for attr in attributes:
            current = getattr(module, attr, None)
            if current is None or isinstance(current, FunctionActivation):
                continue
            if isinstance(current, targets[0]) or current is targets[1] or type(current).__name__.lower().startswith(kind):
                module.__dict__.setdefault(_SLOT, {})[attr] = current
                replacement: Any = FunctionActivation(activation) if isinstance(current, nn.Module) else activation
                setattr(module, attr, replacement)
                patched += 1
    return patched


def restore(model: nn.Module) -> int:
    """Undo `patch_dense_swiglu`, `patch_grouped_experts` and `patch_activation_slots`."""
    restored = 0
    for module in model.modules():
        if hasattr(module, _ORIGINAL):
            original = module.__dict__.pop(_ORIGINAL)
            module.__dict__.pop("forward", None)                 # back to the class's own forward ...
            if getattr(original, "__func__", None) is not type(module).forward:
                module.forward = original                        # ... unless the instance already carried its own
            restored += 1
        slots = module.__dict__.pop(_SLOT, None)
        if slots:
            for attr, original in slots.items():
                setattr(module, attr, original)
                restored += 1
    return restored


__all__ = ["FunctionActivation", "FusedGateUpFeedForward", "dense_swiglu_modules", "fuse_gate_up_projections",
           "gated_mlp_activation",
           "patch_activation_slots", "patch_dense_swiglu", "patch_grouped_experts", "restore", "run_grouped_experts"]
