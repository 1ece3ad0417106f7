"""Gate / up projection with the SwiGLU in its epilogue: `swish(x @ w_gate.T) * (x @ w_up.T)` in one kernel.

The step before the activation at the two feed-forward sites: the fused gate / up feed-forward
(reference: src/sfu_repro/torchtitan/plugin.py:238-239, `w_out(activation_packed(w_in(x)))`) and the routed experts
(reference: plugin.py:294-310, two `_grouped_mm` and `activation_mul`).  There the `[rows, 2 hidden]` products are written
by the matrix product and read back by the activation kernel; here each product tile is rounded to bf16 in registers and
goes through the same packed polynomial program (`fpt_swish_mul`) before anything is stored, so the result equals the
two-step path applied to this kernel's own products bit for bit and the intermediate never exists.

`gate_up_swiglu` is the plain forward; a backward pass needs the products themselves (`raw=True` returns them as
`[rows, 2 hidden]`).  `gate_up_swiglu_recompute` is the differentiable form: it keeps only x and the weights and recomputes
the products in the backward pass (see `sfu_repro.adapters` for where each is used).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_VP = ctypes.c_void_p


def gate_up_swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, *, group_ends: torch.Tensor | None = None,
                   degree: int = 3, coeff_source: str = "current", raw: bool = False) -> torch.Tensor:
    """x `[..., dim]`; w_gate, w_up `[hidden, dim]`, or `[groups, hidden, dim]` with `group_ends` (int32, on the device,
    cumulative row counts: the `offs` of `torch._grouped_mm`) for rows sorted by group.  All bf16, rows contiguous.
    Returns `[..., hidden]` (`raw=True`: `[..., 2 hidden]` = the two products side by side, no activation).  degree 3 is
    the cubic program of the B1 / B4 sites, degree 0 the special-function twin.  Rows past the last group end are left
    as allocated (unwritten), like the rows a grouped matrix product does not own."""
    from .sfu_repro.fa4 import _status_for
    if not (x.is_cuda and w_gate.is_cuda and w_up.is_cuda):
        raise RuntimeError("x, w_gate and w_up must be CUDA tensors")
    if not (x.device == w_gate.device == w_up.device):
        raise RuntimeError("x, w_gate and w_up must be on the same device")
    if not (x.dtype == w_gate.dtype == w_up.dtype == torch.bfloat16):
        raise RuntimeError("x, w_gate and w_up must be bfloat16")
    if w_gate.shape != w_up.shape or w_gate.stride() != w_up.stride() or w_gate.dim() not in (2, 3):
        raise RuntimeError("w_gate and w_up must be [hidden, dim] or [groups, hidden, dim] with the same shape and strides")
    grouped = w_gate.dim() == 3
    if grouped != (group_ends is not None):
        raise RuntimeError("group_ends goes with [groups, hidden, dim] weights, and only with them")
    hidden, dim = w_gate.shape[-2:]
    if x.shape[-1] != dim:
        raise RuntimeError(f"x has {x.shape[-1]} columns, the weights want {dim}")
    if hidden % 128 or dim % 8:
        raise RuntimeError("hidden must be a multiple of 128 and dim a multiple of 8")
    if coeff_source not in ("current", "sollya"):
        raise ValueError(f"unknown coefficient source {coeff_source!r}")
    if w_gate.stride(-1) != 1:
        raise RuntimeError("weight rows must be contiguous")
    x2 = x.reshape(-1, dim)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < dim):
        x2 = x2.contiguous()
    groups = w_gate.shape[0] if grouped else 1
    if grouped:
        if group_ends.dtype != torch.int32 or group_ends.device != x.device or group_ends.numel() != groups or not group_ends.is_contiguous():
            raise RuntimeError("group_ends must be a contiguous int32 tensor of one entry per group on x's device")
        if groups > 256:
            raise RuntimeError("at most 256 groups")
    rows = x2.shape[0]
    width = 2 * hidden if raw else hidden
    out = torch.empty((rows, width), dtype=torch.bfloat16, device=x.device)
    if rows:
        state = _status_for(x.device)
        state.poll()
        lib = _lib.load()
        with torch.cuda.device(x.device):
            stream = _VP(torch.cuda.current_stream(x.device).cuda_stream)
            rc = lib.fpt_gate_up_swiglu(_VP(out.data_ptr()), _VP(x2.data_ptr()), _VP(w_gate.data_ptr()), _VP(w_up.data_ptr()),
                                        rows, dim, hidden, x2.stride(0) if rows > 1 else dim, w_gate.stride(-2),
                                        w_gate.stride(0) if grouped else 0, width,
                                        _VP(group_ends.data_ptr()) if grouped else None, groups, int(degree),
                                        1 if coeff_source == "sollya" else 0, 1 if raw else 0, _VP(state.word.data_ptr()), stream)
        _lib.check("fpt_gate_up_swiglu", rc)
        state.after_launch("fpt_gate_up_swiglu")
    return out.reshape(*x.shape[:-1], width)


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, *, group_ends: torch.Tensor | None = None) -> torch.Tensor:
    """`x @ weight.T` per group with the same kernel: weight `[out, dim]` or `[groups, out, dim]` (out a multiple of 256) is
    taken as two halves of output columns, which is exactly what the kernel's raw epilogue stores side by side.  The
    projection after the activation of the routed experts (reference: src/sfu_repro/torchtitan/plugin.py:308-310, the third
    `_grouped_mm`), where rows are already sorted by group."""
    half = weight.shape[-2] // 2
    if weight.shape[-2] % 256:
        raise RuntimeError("the output width must be a multiple of 256")
    return gate_up_swiglu(x, weight[..., :half, :], weight[..., half:, :], group_ends=group_ends, raw=True)


# ---- dispatcher operators (usable under torch.compile; differentiable by recomputation) -------------------------------
#   fpt_gate_up::swiglu(x, w_gate, w_up, degree, coeff_source_id)   the fused forward
#   fpt_gate_up::products(x, w_gate, w_up)                          [gate | up], the kernel's raw epilogue
# The backward of `swiglu` recomputes the two products with the same kernel (one more projection per layer and step instead
# of a saved [rows, 2 hidden] activation), applies the packed SwiGLU backward kernel to them and leaves the two matrix
# products of the projection's own backward to the library.
_library = torch.library.Library("fpt_gate_up", "DEF")
_library.define("swiglu(Tensor x, Tensor w_gate, Tensor w_up, int degree, int coeff_source_id) -> Tensor")
_library.define("products(Tensor x, Tensor w_gate, Tensor w_up) -> Tensor")
_SOURCES = ("current", "sollya")
_library.impl("swiglu", lambda x, wg, wu, degree, source: gate_up_swiglu(x, wg, wu, degree=degree, coeff_source=_SOURCES[source]), "CUDA")
_library.impl("products", lambda x, wg, wu: gate_up_swiglu(x, wg, wu, raw=True), "CUDA")
torch.library.register_fake("fpt_gate_up::swiglu", lambda x, wg, wu, degree, source: x.new_empty((*x.shape[:-1], wg.shape[-2])),
                            lib=_library)
torch.library.register_fake("fpt_gate_up::products", lambda x, wg, wu: x.new_empty((*x.shape[:-1], 2 * wg.shape[-2])),
                            lib=_library)


def _setup_context(ctx, inputs, output):
    x, w_gate, w_up, ctx.degree, ctx.source = inputs
    ctx.save_for_backward(x, w_gate, w_up)


def _backward(ctx, grad_out):
    from . import spline_ops
    x, w_gate, w_up = ctx.saved_tensors
    hidden, dim = w_gate.shape
    packed = torch.ops.fpt_gate_up.products(x, w_gate, w_up).reshape(-1, 2 * hidden)
    grad_packed = spline_ops.swish_mul_packed_bwd_variant(grad_out.reshape(-1, hidden).contiguous(), packed, ctx.degree, ctx.source)
    grad_gate, grad_up = grad_packed[:, :hidden], grad_packed[:, hidden:]
    x2 = x.reshape(-1, dim)
    grad_x = grad_w_gate = grad_w_up = None
    if ctx.needs_input_grad[0]:
        grad_x = (grad_gate @ w_gate + grad_up @ w_up).reshape(x.shape)
    if ctx.needs_input_grad[1]:
        grad_w_gate = grad_gate.t() @ x2
    if ctx.needs_input_grad[2]:
        grad_w_up = grad_up.t() @ x2
    return grad_x, grad_w_gate, grad_w_up, None, None


torch.library.register_autograd("fpt_gate_up::swiglu", _backward, setup_context=_setup_context, lib=_library)


def gate_up_swiglu_recompute(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, *, degree: int = 3,
                             coeff_source: str = "current") -> torch.Tensor:
    """The dense fused forward as a differentiable dispatcher operator: nothing of size [rows, 2 hidden] is kept for the
    backward pass, which recomputes the two products instead."""
    return torch.ops.fpt_gate_up.swiglu(x, w_gate, w_up, int(degree), _SOURCES.index(coeff_source))


__all__ = ["gate_up_swiglu", "gate_up_swiglu_recompute", "grouped_linear"]
