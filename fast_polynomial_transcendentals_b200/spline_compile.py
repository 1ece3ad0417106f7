"""Dispatcher-level (``torch.compile``-safe) surface of the polynomial activations.

Mirrors the reference's ``spline_compile`` module (reference: autonumerics_zero/spline_ops/spline_compile.py:52-238
for the ``spline_ops::*`` dispatcher operators with fakes and autograd, :268-600 for the ``spline_compile::*``
operators, :603-720 for the factories): same operator names and schemas, same factories, same ``__name__`` /
``__spline_op__`` tags that ``sfu_repro.activations`` checks, same environment switch
``SPLINE_COMPILE_DISABLE_FUSED_SWIGLU``.

The operators are defined once from a table instead of one hand-written block each; every implementation is a call
into ``spline_ops`` (ctypes -> ``libfpt_b200.so``).  The ``spline_ops::`` namespace is the reference extension's: load
either that extension or this module in one process, not both.
"""
from __future__ import annotations

import os
from functools import lru_cache

import torch

from . import spline_ops as _ops

_COEFF_SOURCE_TO_ID = {"current": 0, "sollya": 1}


def _coeff_source_id(coeff_source: str) -> int:
    try:
        return _COEFF_SOURCE_TO_ID[coeff_source]
    except KeyError as exc:
        raise ValueError(
            f"Unknown coeff_source '{coeff_source}'. Expected one of: {tuple(_COEFF_SOURCE_TO_ID)}") from exc


def _env_flag(name: str, default: bool = False) -> bool:
    value = os.environ.get(name)
    return default if value is None else value.lower() in ("1", "true", "yes", "on")


def _like(index=0):
    return lambda *args: torch.empty_like(args[index])


def _halved(packed, *_):
    return packed.new_empty((*packed.shape[:-1], packed.shape[-1] // 2))


_lib = torch.library.Library("spline_ops", "FRAGMENT")
_lib2 = torch.library.Library("spline_compile", "FRAGMENT")

# (library, name, schema tail, implementation, fake)
_OPS = [
    (_lib, "sigmoid_fwd", "(Tensor x) -> Tensor", _ops.sigmoid_fwd, _like()),
    (_lib, "tanh_fwd", "(Tensor x) -> Tensor", _ops.tanh_fwd, _like()),
    (_lib, "swish_fwd", "(Tensor x) -> Tensor", _ops.swish_fwd, _like()),
    (_lib, "sigmoid_bwd", "(Tensor grad_out, Tensor x) -> Tensor", _ops.sigmoid_bwd, _like(1)),
    (_lib, "tanh_bwd", "(Tensor grad_out, Tensor x) -> Tensor", _ops.tanh_bwd, _like(1)),
    (_lib, "swish_bwd", "(Tensor grad_out, Tensor x) -> Tensor", _ops.swish_bwd, _like(1)),
    (_lib, "sigmoid_bwd_alg", "(Tensor grad_out, Tensor y) -> Tensor", _ops.sigmoid_bwd_alg, _like(1)),
    (_lib, "tanh_bwd_alg", "(Tensor grad_out, Tensor y) -> Tensor", _ops.tanh_bwd_alg, _like(1)),
    (_lib, "swish_variant_fwd", "(Tensor x, int degree, int coeff_source_id) -> Tensor", _ops.swish_fwd_variant, _like()),
    (_lib, "swish_variant_bwd", "(Tensor grad_out, Tensor x, int degree, int coeff_source_id) -> Tensor",
     _ops.swish_bwd_variant, _like(1)),
    (_lib, "swish_mul_variant_fwd", "(Tensor gate, Tensor up, int degree, int coeff_source_id) -> Tensor",
     _ops.swish_mul_fwd_variant, _like(1)),
    (_lib, "swish_mul_variant_bwd", "(Tensor grad_out, Tensor gate, Tensor up, int degree, int coeff_source_id) -> Tensor[]",
     _ops.swish_mul_bwd_variant, lambda go, gate, up, *_: [torch.empty_like(gate), torch.empty_like(up)]),
    (_lib, "swish_mul_packed_variant_fwd", "(Tensor packed, int degree, int coeff_source_id) -> Tensor",
     _ops.swish_mul_packed_fwd_variant, _halved),
    (_lib, "swish_mul_packed_native_fwd", "(Tensor packed, int coeff_source_id) -> Tensor",
     lambda packed, src: _ops.swish_mul_packed_fwd_variant(packed, 0, src), _halved),
    (_lib, "swish_mul_packed_native_bwd_fwd", "(Tensor packed, int degree, int coeff_source_id) -> Tensor",
     _ops.swish_mul_packed_fwd_variant, _halved),
    (_lib, "swish_mul_packed_variant_bwd", "(Tensor grad_out, Tensor packed, int degree, int coeff_source_id) -> Tensor",
     _ops.swish_mul_packed_bwd_variant, _like(1)),
    (_lib2, "gelu_fwd", "(Tensor x) -> Tensor", _ops.gelu_fwd, _like()),
    (_lib2, "gelu_bwd", "(Tensor grad_out, Tensor x) -> Tensor", _ops.gelu_bwd, _like(1)),
    (_lib2, "gelu_variant_fwd", "(Tensor x, int degree, int coeff_source_id) -> Tensor", _ops.gelu_fwd_variant, _like()),
    (_lib2, "gelu_variant_bwd", "(Tensor grad_out, Tensor x, int degree, int coeff_source_id) -> Tensor",
     _ops.gelu_bwd_variant, _like(1)),
]

for _library, _name, _schema, _impl, _fake in _OPS:
    _library.define(_name + _schema)
    _library.impl(_name, _impl, "CUDA")
    torch.library.register_fake(f"{_library.ns}::{_name}", _fake, lib=_library)

_so = torch.ops.spline_ops
_sc = torch.ops.spline_compile


def _autograd(qualname: str, n_tensor_inputs: int, save: str, backward):
    """save: 'inputs' keeps the tensor inputs, 'output' keeps the result (algebraic gradients)."""
    def setup_context(ctx, inputs, output):
        ctx.extra = tuple(inputs[n_tensor_inputs:])
        ctx.save_for_backward(*(inputs[:n_tensor_inputs] if save == "inputs" else (output,)))

    def bwd(ctx, grad_out):
        grads = backward(grad_out.contiguous(), *ctx.saved_tensors, *ctx.extra)
        grads = tuple(grads) if isinstance(grads, (tuple, list)) else (grads,)
        return (*grads, *([None] * len(ctx.extra))) if len(grads) + len(ctx.extra) > 1 else grads[0]

    torch.library.register_autograd(qualname, bwd, setup_context=setup_context)


# gradients: which operator computes them (reference: spline_ops.cpp:1933-2183 and spline_compile.py:100-238, 437-556)
_autograd("spline_ops::sigmoid_fwd", 1, "output", lambda go, y: _so.sigmoid_bwd_alg(go, y))
_autograd("spline_ops::tanh_fwd", 1, "output", lambda go, y: _so.tanh_bwd_alg(go, y))
_autograd("spline_ops::swish_fwd", 1, "inputs", lambda go, x: _so.swish_bwd(go, x))
_autograd("spline_ops::swish_variant_fwd", 1, "inputs", lambda go, x, d, s: _so.swish_variant_bwd(go, x, d, s))
_autograd("spline_ops::swish_mul_variant_fwd", 2, "inputs", lambda go, g, u, d, s: _so.swish_mul_variant_bwd(go, g, u, d, s))
_autograd("spline_ops::swish_mul_packed_variant_fwd", 1, "inputs",
          lambda go, p, d, s: _so.swish_mul_packed_variant_bwd(go, p, d, s))
_autograd("spline_ops::swish_mul_packed_native_fwd", 1, "inputs",
          lambda go, p, s: _so.swish_mul_packed_variant_bwd(go, p, 0, s))
_autograd("spline_ops::swish_mul_packed_native_bwd_fwd", 1, "inputs",
          lambda go, p, d, s: _so.swish_mul_packed_variant_bwd(go, p, 0, s))   # polynomial forward, native backward
_autograd("spline_compile::gelu_fwd", 1, "inputs", lambda go, x: _sc.gelu_bwd(go, x))
_autograd("spline_compile::gelu_variant_fwd", 1, "inputs", lambda go, x, d, s: _sc.gelu_variant_bwd(go, x, d, s))


# ---- public API: drop-in activations ------------------------------------------------------------------

def spline_silu(x):
    """Polynomial SiLU (degree 3), differentiable, opaque to torch.compile."""
    return _so.swish_fwd(x)


def spline_sigmoid(x):
    return _so.sigmoid_fwd(x)


def spline_tanh(x):
    return _so.tanh_fwd(x)


def spline_gelu(x):
    return _sc.gelu_fwd(x)


@lru_cache(maxsize=None)
def make_spline_silu(degree: int | None = None, coeff_source: str = "current"):
    resolved_degree = 3 if degree is None else int(degree)
    source_id = _coeff_source_id(coeff_source)

    def activation(x):
        return _so.swish_variant_fwd(x, resolved_degree, source_id)

    activation.__name__ = ("spline_silu_d3_current_cpp" if resolved_degree == 3 and source_id == 0
                           else f"spline_silu_d{resolved_degree}_{coeff_source}")
    return activation


@lru_cache(maxsize=None)
def make_spline_silu_mul(degree: int | None = None, coeff_source: str = "current"):
    resolved_degree = 3 if degree is None else int(degree)
    source_id = _coeff_source_id(coeff_source)
    if source_id != 0 or _env_flag("SPLINE_COMPILE_DISABLE_FUSED_SWIGLU"):
        activation = make_spline_silu(resolved_degree, coeff_source)

        def activation_mul(gate, up):
            return activation(gate.contiguous()) * up.contiguous()

        activation_mul.__name__ = f"spline_silu_mul_d{resolved_degree}_{coeff_source}"
        return activation_mul

    def activation_mul(gate, up):
        return _so.swish_mul_variant_fwd(gate.contiguous(), up.contiguous(), resolved_degree, source_id)

    activation_mul.__name__ = f"spline_silu_mul_d{resolved_degree}_{coeff_source}_fused"
    activation_mul.__spline_op__ = "spline_ops::swish_mul_variant_fwd"
    return activation_mul


@lru_cache(maxsize=None)
def make_spline_silu_packed(degree: int | None = None, coeff_source: str = "current", backward_impl: str = "matched"):
    resolved_degree = 3 if degree is None else int(degree)
    source_id = _coeff_source_id(coeff_source)
    if backward_impl not in ("matched", "native"):
        raise ValueError(f"Unknown packed SwiGLU backward_impl '{backward_impl}'. Expected one of: matched, native")
    if source_id != 0 or _env_flag("SPLINE_COMPILE_DISABLE_FUSED_SWIGLU"):
        activation_mul = make_spline_silu_mul(resolved_degree, coeff_source)

        def activation_packed(packed):
            gate, up = packed.chunk(2, dim=-1)
            poly_out = activation_mul(gate, up)
            if backward_impl == "matched":
                return poly_out
            native_out = torch.nn.functional.silu(gate) * up      # straight-through: polynomial value, native gradient
            return poly_out.detach() + (native_out - native_out.detach())

        activation_packed.__name__ = f"spline_silu_packed_d{resolved_degree}_{coeff_source}"
        return activation_packed
    matched = backward_impl == "matched"
    packed_op = _so.swish_mul_packed_variant_fwd if matched else _so.swish_mul_packed_native_bwd_fwd

    def activation_packed(packed):
        return packed_op(packed.contiguous(), resolved_degree, source_id)

    activation_packed.__name__ = f"spline_silu_packed_d{resolved_degree}_{coeff_source}_{backward_impl}_bwd_fused"
    activation_packed.__spline_op__ = ("spline_ops::swish_mul_packed_variant_fwd" if matched
                                       else "spline_ops::swish_mul_packed_native_bwd_fwd")
    return activation_packed


@lru_cache(maxsize=None)
def make_native_silu_packed():
    def activation_packed(packed):
        return _so.swish_mul_packed_native_fwd(packed.contiguous(), 0)

    activation_packed.__name__ = "native_silu_packed_fused"
    activation_packed.__spline_op__ = "spline_ops::swish_mul_packed_native_fwd"
    return activation_packed


@lru_cache(maxsize=None)
def make_spline_gelu(degree: int | None = None, coeff_source: str = "current"):
    resolved_degree = 5 if degree is None else int(degree)
    source_id = _coeff_source_id(coeff_source)
    if resolved_degree == 5 and source_id == 0:
        return spline_gelu

    def activation(x):
        return _sc.gelu_variant_fwd(x, resolved_degree, source_id)

    activation.__name__ = f"spline_gelu_d{resolved_degree}_{coeff_source}"
    return activation
