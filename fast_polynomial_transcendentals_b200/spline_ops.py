"""The reference's ``spline_ops`` operator surface on top of the C ABI.

Same op names, argument order, defaults, output allocation and error behaviour
as the reference's pybind module (reference:
autonumerics_zero/spline_ops/spline_ops.cpp:2285-2452; argument checks
:293-298, :1647-1649, :1671-1686), implemented as thin Python functions that
validate torch CUDA tensors, allocate the output and call
``libfpt_b200.so`` on the current stream of the tensor's device.

The hot element-wise operators (unary, gradient product, the four SwiGLU forms) go through a compiled PyTorch
binding when it has been built (``_fpt_torch``: checks, allocation, device guard and the C-ABI call in C++; the same
functions are also registered as dispatcher operators ``torch.ops.fpt_b200.*``); everything else, and those six when the
binding is absent, goes through ``ctypes`` on the same library.  Either way the work is done by ``libfpt_b200.so``.

Differences kept on purpose:
  * the call runs under a device guard for the input tensor's device (the
    reference assumes the current device already matches);
  * element counts are 64-bit all the way down (the reference narrows
    ``numel()`` to ``int`` for the flat ops).
Errors are ``RuntimeError`` like ``TORCH_CHECK``.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import BF16, BWD, FN_GELU, FN_SIGMOID, FN_SWISH, FN_TANH, FP16, FWD

try:                                    # the compiled binding (built by build.py next to the CUDA library)
    _lib.load()
    from . import _fpt_torch as _ext
except ImportError:
    _ext = None


def binding_kind() -> str:
    """How the hot element-wise operators reach the CUDA library in this process."""
    return "compiled torch extension (_fpt_torch)" if _ext is not None else "ctypes"


_FUNCTIONS = {"sigmoid": FN_SIGMOID, "tanh": FN_TANH, "swish": FN_SWISH, "gelu": FN_GELU}
_DEFAULT_DEGREE = {("sigmoid", "fwd"): 3, ("sigmoid", "bwd"): 4, ("tanh", "fwd"): 3, ("tanh", "bwd"): 4,
                   ("swish", "fwd"): 3, ("swish", "bwd"): 4, ("gelu", "fwd"): 5, ("gelu", "bwd"): 5}


def _check_input(x: torch.Tensor, name: str) -> None:
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"{name} must be float16 or bfloat16")


def _check_fp16(x: torch.Tensor, name: str) -> None:
    _check_input(x, name)
    if x.dtype != torch.float16:
        raise RuntimeError(f"{name} must be float16")


def _dtype_id(x: torch.Tensor) -> int:
    return BF16 if x.dtype == torch.bfloat16 else FP16


def _source(coeff_source_id: int, x: torch.Tensor) -> int:
    if coeff_source_id not in (0, 1):
        raise RuntimeError("coeff_source_id must be 0 (current) or 1 (sollya)")
    if coeff_source_id == 1 and x.dtype != torch.bfloat16:
        raise RuntimeError("FP16 spline kernels only support coeff_source=current")
    return int(coeff_source_id)


def _same(a: torch.Tensor, b: torch.Tensor, an: str, bn: str) -> None:
    """Two tensors of one launch: the kernel indexes both with one element count, reads both as one lane format and
    runs on one device, so all three must agree before anything is launched."""
    if a.dtype != b.dtype:
        raise RuntimeError(f"{an} and {bn} must have the same dtype")
    if a.numel() != b.numel():
        raise RuntimeError(f"{an} and {bn} must have the same number of elements")
    if a.device != b.device:
        raise RuntimeError(f"{an} and {bn} must be on the same device")


class _Guard:
    """Make the tensor's device current for the duration of one launch."""

    __slots__ = ("index", "prev")

    def __init__(self, x: torch.Tensor):
        self.index = x.device.index
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)
        return torch.cuda.current_stream(self.index).cuda_stream

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def _call(name: str, x: torch.Tensor, *args) -> None:
    fn = getattr(_lib.load(), name)
    with _Guard(x) as stream:
        status = fn(*args, stream)
    if status != 0:
        _lib.check(name, status)


# ---- unary / gradient products -------------------------------------------------------------

def _unary(x, function: str, direction: int, degree: int, source: int = 0):
    if _ext is not None and isinstance(x, torch.Tensor):
        return _ext.unary(x, _FUNCTIONS[function], direction, degree, source)
    _check_input(x, "x")
    out = torch.empty_like(x)
    try:
        _call("fpt_unary", x, out.data_ptr(), x.data_ptr(), x.numel(), _FUNCTIONS[function], direction, degree,
              _dtype_id(x), source)
    except _lib.FptError as err:
        if err.status == -4:
            which = "forward" if direction == FWD else "backward"
            raise RuntimeError(f"Unsupported {function} {which} degree: {degree}") from None
        raise
    return out


def _binary(grad_out, x, function: str, degree: int, source: int = 0):
    if _ext is not None and isinstance(grad_out, torch.Tensor) and isinstance(x, torch.Tensor):
        return _ext.binary_bwd(grad_out, x, _FUNCTIONS[function], degree, source)
    _check_input(grad_out, "grad_out")
    _check_input(x, "x")
    _same(grad_out, x, "grad_out", "x")
    grad_in = torch.empty_like(x)
    try:
        _call("fpt_binary_bwd", x, grad_in.data_ptr(), grad_out.data_ptr(), x.data_ptr(), x.numel(),
              _FUNCTIONS[function], degree, _dtype_id(x), source)
    except _lib.FptError as err:
        if err.status == -4:
            raise RuntimeError(f"Unsupported {function} backward degree: {degree}") from None
        raise
    return grad_in


def _make_fixed(function: str, direction: str, degree: int):
    if direction == "fwd":
        def op(x):
            return _unary(x, function, FWD, degree)
    else:
        def op(grad_out, x):
            return _binary(grad_out, x, function, degree)
    return op


for _fn in ("sigmoid", "tanh", "swish", "gelu"):
    for _dir in ("fwd", "bwd"):
        globals()[f"{_fn}_{_dir}"] = _make_fixed(_fn, _dir, _DEFAULT_DEGREE[(_fn, _dir)])
        globals()[f"{_fn}_{_dir}"].__doc__ = f"{_fn} {_dir}, default degree {_DEFAULT_DEGREE[(_fn, _dir)]}"
        for _deg in (3, 4, 5, 6):
            globals()[f"{_fn}_{_dir}_d{_deg}"] = _make_fixed(_fn, _dir, _deg)


def sigmoid_fwd_variant(x, degree: int, coeff_source_id: int):
    return _unary(x, "sigmoid", FWD, int(degree), _source(coeff_source_id, x))


def sigmoid_bwd_variant(grad_out, x, degree: int, coeff_source_id: int):
    return _binary(grad_out, x, "sigmoid", int(degree), _source(coeff_source_id, x))


def swish_fwd_variant(x, degree: int, coeff_source_id: int):
    """degree 0 selects the native special-function-unit kernel."""
    return _unary(x, "swish", FWD, int(degree), _source(coeff_source_id, x))


def swish_bwd_variant(grad_out, x, degree: int, coeff_source_id: int):
    return _binary(grad_out, x, "swish", int(degree), _source(coeff_source_id, x))


def gelu_fwd_variant(x, degree: int, coeff_source_id: int):
    return _unary(x, "gelu", FWD, int(degree), _source(coeff_source_id, x))


def gelu_bwd_variant(grad_out, x, degree: int, coeff_source_id: int):
    return _binary(grad_out, x, "gelu", int(degree), _source(coeff_source_id, x))


def _alg(grad_out, y, function: str):
    _check_input(grad_out, "grad_out")
    _check_input(y, "x")
    _same(grad_out, y, "grad_out", "x")
    grad_in = torch.empty_like(y)
    _call("fpt_bwd_algebraic", y, grad_in.data_ptr(), grad_out.data_ptr(), y.data_ptr(), y.numel(),
          _FUNCTIONS[function], _dtype_id(y))
    return grad_in


def sigmoid_bwd_alg(grad_out, y):
    """grad_in = grad_out * y * (1 - y) from the saved forward output."""
    return _alg(grad_out, y, "sigmoid")


def tanh_bwd_alg(grad_out, y):
    """grad_in = grad_out * (1 - y^2) from the saved forward output."""
    return _alg(grad_out, y, "tanh")


# ---- FP16-only composites (reference: spline_ops.cpp:1547-1575 hybrid fwd, :1862-1864 hybrid bwd, :1866-1926) ----

def _check_fp16_only(x: torch.Tensor, name: str) -> None:
    _check_input(x, name)
    if x.dtype != torch.float16:
        raise RuntimeError(f"{name} must be float16 (no BF16 support for this op)")


def _hybrid_fwd(function: str):
    def op(x):
        _check_fp16_only(x, "x")
        out = torch.empty_like(x)
        _call("fpt_unary_hybrid", x, out.data_ptr(), x.data_ptr(), x.numel(), _FUNCTIONS[function])
        return out
    op.__name__ = f"{function}_fwd_hybrid"
    op.__doc__ = f"{function} forward, one packed word in four on the SFU and three on the D3 polynomial."
    return op


def _hybrid_bwd(function: str):
    def op(grad_out, x):
        _check_fp16_only(grad_out, "grad_out")
        _check_fp16_only(x, "x")
        _same(grad_out, x, "grad_out", "x")
        grad_in = torch.empty_like(x)
        _call("fpt_binary_bwd_hybrid", x, grad_in.data_ptr(), grad_out.data_ptr(), x.data_ptr(), x.numel(),
              _FUNCTIONS[function])
        return grad_in
    op.__name__ = f"{function}_bwd_hybrid"
    op.__doc__ = f"grad_out * d{function}/dx, one packed word in four on the SFU and three on the D4 polynomial."
    return op


def _fused(function: str):
    def op(x, grad_out):
        _check_fp16_only(x, "x")
        _check_fp16_only(grad_out, "grad_out")
        _same(x, grad_out, "x", "grad_out")
        y, grad_in = torch.empty_like(x), torch.empty_like(x)
        _call("fpt_fused_fwd_bwd", x, y.data_ptr(), grad_in.data_ptr(), x.data_ptr(), grad_out.data_ptr(), x.numel(),
              _FUNCTIONS[function])
        return [y, grad_in]
    op.__name__ = f"{function}_fused"
    op.__doc__ = f"[{function}_D3(x), grad_out * derivative] in one pass over x."
    return op


_DERIV_ALGEBRAIC, _DERIV_POLY, _DERIV_SHARED_SIGMOID = 0, 1, 2


def _fwd_deriv(function: str, variant: int, name: str):
    def op(x):
        _check_fp16_only(x, "x")
        y, dy = torch.empty_like(x), torch.empty_like(x)
        _call("fpt_fwd_deriv", x, y.data_ptr(), dy.data_ptr(), x.data_ptr(), x.numel(), _FUNCTIONS[function], variant)
        return [y, dy]
    op.__name__ = name
    op.__doc__ = "[y, dy/dx]: the forward value and the derivative saved for a multiply-only backward."
    return op


sigmoid_fwd_hybrid, tanh_fwd_hybrid, swish_fwd_hybrid = (_hybrid_fwd(f) for f in ("sigmoid", "tanh", "swish"))
sigmoid_bwd_hybrid, tanh_bwd_hybrid, swish_bwd_hybrid = (_hybrid_bwd(f) for f in ("sigmoid", "tanh", "swish"))
sigmoid_fused, tanh_fused, swish_fused = (_fused(f) for f in ("sigmoid", "tanh", "swish"))
sigmoid_fwd_deriv_alg = _fwd_deriv("sigmoid", _DERIV_ALGEBRAIC, "sigmoid_fwd_deriv_alg")
sigmoid_fwd_deriv_poly = _fwd_deriv("sigmoid", _DERIV_POLY, "sigmoid_fwd_deriv_poly")
tanh_fwd_deriv_alg = _fwd_deriv("tanh", _DERIV_ALGEBRAIC, "tanh_fwd_deriv_alg")
tanh_fwd_deriv_poly = _fwd_deriv("tanh", _DERIV_POLY, "tanh_fwd_deriv_poly")
swish_fwd_deriv = _fwd_deriv("swish", _DERIV_SHARED_SIGMOID, "swish_fwd_deriv")
swish_fwd_deriv_poly = _fwd_deriv("swish", _DERIV_POLY, "swish_fwd_deriv_poly")


def multiply(a, b):
    """a * b, one rounding per lane (the backward of the forward-with-derivative ops: grad_out * saved dy)."""
    _check_input(a, "a")
    _check_input(b, "b")
    _same(a, b, "a", "b")
    out = torch.empty_like(a)
    _call("fpt_multiply", a, out.data_ptr(), a.data_ptr(), b.data_ptr(), a.numel(), _dtype_id(a))
    return out


# ---- SwiGLU --------------------------------------------------------------------------------

def swish_mul_fwd_variant(gate, up, degree: int, coeff_source_id: int):
    if _ext is not None and isinstance(gate, torch.Tensor) and isinstance(up, torch.Tensor):
        return _ext.swish_mul(gate, up, int(degree), int(coeff_source_id))
    _check_input(gate, "gate")
    _check_input(up, "up")
    _same(gate, up, "gate", "up")
    source = _source(coeff_source_id, gate)
    out = torch.empty_like(up)
    try:
        _call("fpt_swish_mul", gate, out.data_ptr(), gate.data_ptr(), up.data_ptr(), gate.numel(), int(degree),
              _dtype_id(gate), source)
    except _lib.FptError as err:
        if err.status == -4:
            raise RuntimeError(f"Unsupported swish_mul forward degree: {degree}") from None
        raise
    return out


def swish_mul_bwd_variant(grad_out, gate, up, degree: int, coeff_source_id: int):
    if _ext is not None and all(isinstance(t, torch.Tensor) for t in (grad_out, gate, up)):
        return list(_ext.swish_mul_bwd(grad_out, gate, up, int(degree), int(coeff_source_id)))
    for t, n in ((grad_out, "grad_out"), (gate, "gate"), (up, "up")):
        _check_input(t, n)
    if not (grad_out.dtype == gate.dtype == up.dtype):
        raise RuntimeError("grad_out, gate, and up must have the same dtype")
    if not (grad_out.numel() == gate.numel() == up.numel()):
        raise RuntimeError("grad_out, gate, and up must have the same number of elements")
    if not (grad_out.device == gate.device == up.device):
        raise RuntimeError("grad_out, gate, and up must be on the same device")
    source = _source(coeff_source_id, gate)
    grad_gate, grad_up = torch.empty_like(gate), torch.empty_like(up)
    try:
        _call("fpt_swish_mul_bwd", gate, grad_gate.data_ptr(), grad_up.data_ptr(), grad_out.data_ptr(),
              gate.data_ptr(), up.data_ptr(), gate.numel(), int(degree), _dtype_id(gate), source)
    except _lib.FptError as err:
        if err.status == -4:
            raise RuntimeError(f"Unsupported swish_mul backward degree: {degree}") from None
        raise
    return [grad_gate, grad_up]


def _packed_dims(packed):
    if packed.dim() < 1:
        raise RuntimeError("packed gate/up tensor must have at least one dimension")
    width = packed.size(-1)
    if width % 2:
        raise RuntimeError("packed gate/up last dimension must be even")
    hidden = width // 2
    if hidden % 2:
        raise RuntimeError("packed SwiGLU hidden size must be even")
    return width, hidden


def swish_mul_packed_fwd_variant(packed, degree: int, coeff_source_id: int):
    """packed [..., 2H] = [gate | up]  ->  [..., H]."""
    if _ext is not None and isinstance(packed, torch.Tensor):
        return _ext.swish_mul_packed(packed, int(degree), int(coeff_source_id))
    _check_input(packed, "packed")
    width, hidden = _packed_dims(packed)
    source = _source(coeff_source_id, packed)
    out = torch.empty(*packed.shape[:-1], hidden, dtype=packed.dtype, device=packed.device)
    if packed.numel() == 0:
        return out
    rows = packed.numel() // width
    try:
        _call("fpt_swish_mul_packed", packed, out.data_ptr(), packed.data_ptr(), rows, hidden, int(degree),
              _dtype_id(packed), source)
    except _lib.FptError as err:
        if err.status == -4:
            raise RuntimeError(f"Unsupported packed swish_mul forward degree: {degree}") from None
        raise
    return out


def swish_mul_packed_bwd_variant(grad_out, packed, degree: int, coeff_source_id: int):
    if _ext is not None and isinstance(grad_out, torch.Tensor) and isinstance(packed, torch.Tensor):
        return _ext.swish_mul_packed_bwd(grad_out, packed, int(degree), int(coeff_source_id))
    _check_input(grad_out, "grad_out")
    _check_input(packed, "packed")
    if grad_out.dtype != packed.dtype:
        raise RuntimeError("grad_out and packed must have the same dtype")
    if grad_out.device != packed.device:
        raise RuntimeError("grad_out and packed must be on the same device")
    width, hidden = _packed_dims(packed)
    if grad_out.numel() * 2 != packed.numel() or (grad_out.dim() and grad_out.size(-1) != hidden):
        raise RuntimeError("grad_out must match the packed tensor with its last dimension halved")
    source = _source(coeff_source_id, packed)
    grad_packed = torch.empty_like(packed)
    if packed.numel() == 0:
        return grad_packed
    rows = packed.numel() // width
    try:
        _call("fpt_swish_mul_packed_bwd", packed, grad_packed.data_ptr(), grad_out.data_ptr(), packed.data_ptr(),
              rows, hidden, int(degree), _dtype_id(packed), source)
    except _lib.FptError as err:
        if err.status == -4:
            raise RuntimeError(f"Unsupported packed swish_mul backward degree: {degree}") from None
        raise
    return grad_packed


# ---- paired sin/cos (reference: spline_ops.cpp:325-560) ---------------------------------------

_SINCOS_VARIANTS = {
    "d3_d4_quarter_turn_fp16": 0, "d3_d4_half_turn_fp16": 1, "d5_d4_half_turn_fp16": 2, "d5_d6_half_turn_fp16": 3,
    "d7_d6_half_turn_fp16": 4, "d3_d4_bf16": 5, "d3_d4_quarter_turn_bf16": 6, "d3_d4_half_turn_bf16": 7,
    "d5_d6_half_turn_bf16": 8, "d5_d4_half_turn_fp16_bf16": 9, "native_fp16": 10, "native_bf16": 11,
}


def _sincos(angles, variant: int, out_dtype, iterations: int = 0):
    if not isinstance(angles, torch.Tensor) or not angles.is_cuda:
        raise RuntimeError("angles must be a CUDA tensor")
    if not angles.is_contiguous():
        raise RuntimeError("angles must be contiguous")
    if angles.dtype != torch.float32:
        raise RuntimeError("angles must be float32")
    out = torch.empty((2, *angles.shape), dtype=out_dtype, device=angles.device)
    _call("fpt_sincos", angles, out.data_ptr(), angles.data_ptr(), angles.numel(), variant, iterations)
    return out


def _make_sincos(variant: int, out_dtype, compute: bool):
    if compute:
        def op(angles, iterations):
            if int(iterations) <= 0:
                raise RuntimeError("iterations must be positive")
            return _sincos(angles, variant, out_dtype, int(iterations))
    else:
        def op(angles):
            return _sincos(angles, variant, out_dtype)
    op.__doc__ = "angles fp32 [...] -> [2, ...] (cos first)"
    return op


for _name, _variant in _SINCOS_VARIANTS.items():
    _dtype = torch.bfloat16 if _name.endswith("bf16") else torch.float16
    globals()[f"sincos_{_name}"] = _make_sincos(_variant, _dtype, False)
    globals()[f"sincos_{_name}_compute"] = _make_sincos(_variant, _dtype, True)


# fp32 family: `sincos_<variant>_f32(angles)` and `sincos_<variant>_compute_f32(angles, iterations)`
_SINCOS_F32_VARIANTS = ("native", "d3_d4", "d3_d4_cycle", "d3_d4_magic_bias", "d5_d4_half_turn_ls",
                        "d5_d4_half_turn_sollya", "d5_d4_half_turn_sollya_fast", "d5_d4", "d7_d6")


def _sincos_f32(angles, variant: int, iterations: int = 0):
    if not isinstance(angles, torch.Tensor) or not angles.is_cuda:
        raise RuntimeError("angles must be a CUDA tensor")
    if not angles.is_contiguous():
        raise RuntimeError("angles must be contiguous")
    if angles.dtype != torch.float32:
        raise RuntimeError("angles must be float32")
    out = torch.empty((2, *angles.shape), dtype=torch.float32, device=angles.device)
    _call("fpt_sincos_f32", angles, out.data_ptr(), angles.data_ptr(), angles.numel(), variant, iterations)
    return out


def _make_sincos_f32(variant: int, compute: bool):
    if compute:
        def op(angles, iterations):
            if int(iterations) <= 0:
                raise RuntimeError("iterations must be positive")
            return _sincos_f32(angles, variant, int(iterations))
    else:
        def op(angles):
            return _sincos_f32(angles, variant)
    op.__doc__ = "angles fp32 [...] -> fp32 [2, ...] (cos first)"
    return op


for _variant, _name in enumerate(_SINCOS_F32_VARIANTS):
    globals()[f"sincos_{_name}_f32"] = _make_sincos_f32(_variant, False)
    globals()[f"sincos_{_name}_compute_f32"] = _make_sincos_f32(_variant, True)


# ---- RoPE (reference: spline_ops.cpp:562-1140) -------------------------------------------------

ROPE_HALF_TURN_D5_D6, ROPE_QUARTER_TURN_D3_D4, ROPE_NATIVE, ROPE_CACHED = 0, 1, 2, 3


def _rope_table(parameters, sequence_length: int, kind: int, dtype, name: str, iterations: int = 0):
    if not isinstance(parameters, torch.Tensor) or not parameters.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not parameters.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if parameters.dim() != 1:
        raise RuntimeError(f"{name} must be one-dimensional")
    if parameters.dtype != dtype:
        raise RuntimeError(f"{name} has the wrong dtype")
    if int(sequence_length) <= 0:
        raise RuntimeError("sequence_length must be positive")
    if parameters.numel() == 0 or parameters.numel() % 2:
        raise RuntimeError(f"{name} must contain a positive even number of elements")
    out = torch.empty((2, int(sequence_length), parameters.numel()), dtype=torch.float16, device=parameters.device)
    _call("fpt_rope_table", parameters, out.data_ptr(), parameters.data_ptr(), int(sequence_length),
          parameters.numel(), kind, iterations)
    return out


def rope_sincos_native_fp16(frequencies, sequence_length):
    return _rope_table(frequencies, sequence_length, ROPE_NATIVE, torch.float32, "frequencies")


def rope_sincos_fixed_d3_d4_fp16(phase_increments, sequence_length):
    return _rope_table(phase_increments, sequence_length, ROPE_QUARTER_TURN_D3_D4, torch.int32, "phase_increments")


def rope_sincos_fixed_half_turn_d5_d6_fp16(phase_increments, sequence_length):
    if phase_increments.numel() % 4:
        raise RuntimeError("phase_increments must contain a multiple of four elements")
    return _rope_table(phase_increments, sequence_length, ROPE_HALF_TURN_D5_D6, torch.int32, "phase_increments")


def rope_sincos_native_fp16_compute(frequencies, sequence_length, iterations):
    return _rope_table(frequencies, sequence_length, ROPE_NATIVE, torch.float32, "frequencies", int(iterations))


def rope_sincos_fixed_d3_d4_fp16_compute(phase_increments, sequence_length, iterations):
    return _rope_table(phase_increments, sequence_length, ROPE_QUARTER_TURN_D3_D4, torch.int32, "phase_increments",
                       int(iterations))


def rope_sincos_fixed_half_turn_d5_d6_fp16_compute(phase_increments, sequence_length, iterations):
    return _rope_table(phase_increments, sequence_length, ROPE_HALF_TURN_D5_D6, torch.int32, "phase_increments",
                       int(iterations))


def _rope_table_lut(phase_increments, phase_table, sequence_length, iterations: int = 0):
    if not isinstance(phase_table, torch.Tensor) or not phase_table.is_cuda:
        raise RuntimeError("phase_table must be a CUDA tensor")
    if not phase_table.is_contiguous():
        raise RuntimeError("phase_table must be contiguous")
    if phase_table.dtype != torch.float16:
        raise RuntimeError("phase_table must be float16")
    if phase_table.dim() != 2 or phase_table.size(0) != 128 or phase_table.size(1) != 2:
        raise RuntimeError("phase_table must have shape [128, 2]")
    if not isinstance(phase_increments, torch.Tensor) or not phase_increments.is_cuda:
        raise RuntimeError("phase_increments must be a CUDA tensor")
    if phase_table.device != phase_increments.device:
        raise RuntimeError("phase_table and phase_increments must be on the same CUDA device")
    if not phase_increments.is_contiguous():
        raise RuntimeError("phase_increments must be contiguous")
    if phase_increments.dim() != 1:
        raise RuntimeError("phase_increments must be one-dimensional")
    if phase_increments.dtype != torch.int32:
        raise RuntimeError("phase_increments has the wrong dtype")
    if int(sequence_length) <= 0:
        raise RuntimeError("sequence_length must be positive")
    if phase_increments.numel() == 0 or phase_increments.numel() % 2:
        raise RuntimeError("phase_increments must contain a positive even number of elements")
    out = torch.empty((2, int(sequence_length), phase_increments.numel()), dtype=torch.float16,
                      device=phase_increments.device)
    _call("fpt_rope_table_lut", phase_increments, out.data_ptr(), phase_increments.data_ptr(), phase_table.data_ptr(),
          int(sequence_length), phase_increments.numel(), iterations)
    return out


def rope_sincos_fixed_lut_fp16(phase_increments, phase_table, sequence_length):
    """[2, S, F] fp16 (cos, sin) from a [128, 2] (sin, cos) table and one first-order correction step."""
    return _rope_table_lut(phase_increments, phase_table, sequence_length)


def rope_sincos_fixed_lut_fp16_compute(phase_increments, phase_table, sequence_length, iterations):
    if int(iterations) <= 0:
        raise RuntimeError("iterations must be positive")
    return _rope_table_lut(phase_increments, phase_table, sequence_length, int(iterations))


def _check_rope_qk(q, k, dtype, dtype_name):
    for t, n in ((q, "q"), (k, "k")):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"{n} must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{n} must be contiguous")
        if t.dtype != dtype:
            raise RuntimeError(f"{n} must be {dtype_name}")
        if t.dim() != 4:
            raise RuntimeError(f"{n} must have shape [batch, sequence, heads, head_dim]")
    if q.device != k.device:
        raise RuntimeError("q and k must be on the same CUDA device")
    if q.size(0) != k.size(0):
        raise RuntimeError("q and k batch sizes must match")
    if q.size(1) != k.size(1):
        raise RuntimeError("q and k sequence lengths must match")
    if q.size(3) != k.size(3):
        raise RuntimeError("q and k head dimensions must match")
    if q.size(2) <= 0 or k.size(2) <= 0:
        raise RuntimeError("q and k must contain at least one head")
    if q.size(3) <= 0 or q.size(3) % 8:
        raise RuntimeError("head_dim must be a positive multiple of eight")
    if q.size(0) > 65535:
        raise RuntimeError("batch size is too large for the CUDA grid")


def _rope_apply(q, k, parameters, kind: int, param_dtype, name: str, io_dtype=torch.float16):
    _check_rope_qk(q, k, io_dtype, "float16" if io_dtype == torch.float16 else "bfloat16")
    if not isinstance(parameters, torch.Tensor) or not parameters.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not parameters.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    B, S, Hq, D = q.shape
    Hk = k.size(2)
    if kind == ROPE_CACHED:
        if parameters.dtype != torch.float16:
            raise RuntimeError("rope_table must be float16")
        if parameters.dim() != 3 or tuple(parameters.shape) != (2, S, D // 2):
            raise RuntimeError("rope_table must have shape [2, sequence, head_dim / 2]")
    else:
        if parameters.dim() != 1:
            raise RuntimeError(f"{name} must be one-dimensional")
        if parameters.dtype != param_dtype:
            raise RuntimeError(f"{name} has the wrong dtype")
        if parameters.numel() != D // 2:
            raise RuntimeError(f"{name} must contain head_dim / 2 elements")
    if parameters.device != q.device:
        raise RuntimeError(f"{name} must be on the same CUDA device as q and k")
    q_out = torch.empty((B, Hq, S, D), dtype=q.dtype, device=q.device)
    k_out = torch.empty((B, Hk, S, D), dtype=k.dtype, device=k.device)
    _call("fpt_rope_apply", q, q_out.data_ptr(), k_out.data_ptr(), q.data_ptr(), k.data_ptr(), parameters.data_ptr(),
          B, S, Hq, Hk, D, kind, BF16 if io_dtype == torch.bfloat16 else FP16)
    return [q_out, k_out]


def rope_apply_fixed_half_turn_d5_d6_fp16(q, k, phase_increments):
    """Fused polynomial RoPE + transpose: [B,S,H,D] fp16 -> [B,H,S,D]."""
    return _rope_apply(q, k, phase_increments, ROPE_HALF_TURN_D5_D6, torch.int32, "phase_increments")


def rope_apply_native_fp16(q, k, frequencies):
    return _rope_apply(q, k, frequencies, ROPE_NATIVE, torch.float32, "frequencies")


def rope_apply_cached_fp16(q, k, rope_table):
    return _rope_apply(q, k, rope_table, ROPE_CACHED, torch.float16, "rope_table")


def rope_apply_fixed_half_turn_d5_d6_bf16(q, k, phase_increments):
    """Not in the reference: the same fp16 polynomial rotation around bf16 inputs and outputs, the form a
    bf16 attention consumes."""
    return _rope_apply(q, k, phase_increments, ROPE_HALF_TURN_D5_D6, torch.int32, "phase_increments", torch.bfloat16)


# ---- score-mod evaluators as stand-alone ops (not in the reference's module) --------------------

EXP2_NATIVE, EXP2_HINGE_LEAST_SQUARES, EXP2_HINGE_ENDPOINT = 0, 1, 2


def exp2_fraction(x, variant: int = EXP2_HINGE_LEAST_SQUARES, repeats: int = 1):
    """2^x for fp16 x in [0, 1): native MUFU, or the two-segment hinge with either constant set."""
    _check_fp16(x, "x")
    out = torch.empty_like(x)
    _call("fpt_exp2_fraction", x, out.data_ptr(), x.data_ptr(), x.numel(), int(variant), int(repeats))
    return out



EXP2_FULL_D3, EXP2_FULL_PWL2 = 0, 1


def exp2_full_f32(x, variant: int = EXP2_FULL_D3):
    """2^x for fp32 x <= 127 on the FMA pipe: floor reduction, then a cubic (D3) or a two-piece line (PWL2) in the
    fraction; inputs below -127 give the value at -127."""
    if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
        raise ValueError("x must be a contiguous fp32 CUDA tensor")
    out = torch.empty_like(x)
    _call("fpt_exp2_full_f32", x, out.data_ptr(), x.data_ptr(), x.numel(), int(variant))
    return out


# ---- differentiable entry points (reference: C++ autograd Functions, spline_ops.cpp:1933-2205) ---

class _UnaryAutograd(torch.autograd.Function):
    """y = F(x); backward through the polynomial derivative program of the same degree and source."""

    @staticmethod
    def forward(ctx, x, function, degree, source):
        ctx.save_for_backward(x)
        ctx.spec = (function, degree, source)
        return _unary(x, function, FWD, degree, source)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        function, degree, source = ctx.spec
        return _binary(grad_out.contiguous(), x, function, degree, source), None, None, None


class _AlgebraicAutograd(torch.autograd.Function):
    """sigmoid / tanh with the gradient computed from the saved output."""

    @staticmethod
    def forward(ctx, x, function):
        y = _unary(x, function, FWD, 3)
        ctx.save_for_backward(y)
        ctx.function = function
        return y

    @staticmethod
    def backward(ctx, grad_out):
        (y,) = ctx.saved_tensors
        return _alg(grad_out.contiguous(), y, ctx.function), None


class _SwishMulAutograd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, degree, source):
        ctx.save_for_backward(gate, up)
        ctx.spec = (degree, source)
        return swish_mul_fwd_variant(gate, up, degree, source)

    @staticmethod
    def backward(ctx, grad_out):
        gate, up = ctx.saved_tensors
        grad_gate, grad_up = swish_mul_bwd_variant(grad_out.contiguous(), gate, up, *ctx.spec)
        return grad_gate, grad_up, None, None


def sigmoid_ag(x):
    return _AlgebraicAutograd.apply(x, "sigmoid")


def tanh_ag(x):
    return _AlgebraicAutograd.apply(x, "tanh")


def swish_ag(x):
    """Forward D3, backward D4: the defaults of swish_fwd / swish_bwd."""
    class _Mixed(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t):
            ctx.save_for_backward(t)
            return swish_fwd(t)

        @staticmethod
        def backward(ctx, grad_out):
            (t,) = ctx.saved_tensors
            return swish_bwd(grad_out.contiguous(), t)
    return _Mixed.apply(x)


def swish_ag_variant(x, degree: int, coeff_source_id: int):
    _check_input(x, "x")
    return _UnaryAutograd.apply(x, "swish", int(degree), _source(coeff_source_id, x))


def gelu_ag_variant(x, degree: int, coeff_source_id: int):
    _check_input(x, "x")
    return _UnaryAutograd.apply(x, "gelu", int(degree), _source(coeff_source_id, x))


def swish_mul_ag_variant(gate, up, degree: int, coeff_source_id: int):
    _check_input(gate, "gate")
    return _SwishMulAutograd.apply(gate, up, int(degree), _source(coeff_source_id, gate))
