"""ctypes binding of ``libfpt_b200.so`` -- the only route from Python to the CUDA kernels.

There is no CPU or PyTorch fallback: if the shared library is missing or a call
returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libfpt_b200.so"

FP16, BF16 = 0, 1
SRC_CURRENT, SRC_SOLLYA = 0, 1
FN_SIGMOID, FN_TANH, FN_SWISH, FN_ERF, FN_GELU = range(5)
FWD, BWD = 0, 1

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_u16p = ctypes.POINTER(ctypes.c_uint16)

# name -> argument types; every entry point returns an int status unless noted in _RESTYPES
SIGNATURES: dict[str, list] = {
    "fpt_program_count": [],
    "fpt_program_info": [_int, ctypes.c_char_p, _int, ctypes.POINTER(_int), ctypes.POINTER(_int),
                         ctypes.POINTER(_int), ctypes.POINTER(_int), _u16p, _u16p],
    "fpt_unary": [_vp, _vp, _i64, _int, _int, _int, _int, _int, _vp],
    "fpt_unary_repeat": [_vp, _vp, _i64, _int, _int, _int, _int, _int, _int, _vp],
    "fpt_binary_bwd": [_vp, _vp, _vp, _i64, _int, _int, _int, _int, _vp],
    "fpt_bwd_algebraic": [_vp, _vp, _vp, _i64, _int, _int, _vp],
    "fpt_swish_mul": [_vp, _vp, _vp, _i64, _int, _int, _int, _vp],
    "fpt_swish_mul_bwd": [_vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _int, _vp],
    "fpt_swish_mul_packed": [_vp, _vp, _i64, _i64, _int, _int, _int, _vp],
    "fpt_swish_mul_packed_bwd": [_vp, _vp, _vp, _i64, _i64, _int, _int, _int, _vp],
    "fpt_gate_up_swiglu": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _i64, _int, _int, _int, _vp, _vp],
    "fpt_b3_sigmoid_direct": [_vp, _vp, _vp, _i64, _int, _int, _vp],
    "fpt_b3_sigmoid_direct_variant": [_vp, _vp, _vp, _i64, _int, _int, _int, _vp],
    "fpt_fwd_deriv": [_vp, _vp, _vp, _i64, _int, _int, _vp],
    "fpt_fused_fwd_bwd": [_vp, _vp, _vp, _vp, _i64, _int, _vp],
    "fpt_multiply": [_vp, _vp, _vp, _i64, _int, _vp],
    "fpt_unary_hybrid": [_vp, _vp, _i64, _int, _vp],
    "fpt_binary_bwd_hybrid": [_vp, _vp, _vp, _i64, _int, _vp],
    "fpt_exp2_fraction": [_vp, _vp, _i64, _int, _int, _vp],
    "fpt_exp2_full_f32": [_vp, _vp, _i64, _int, _vp],
    "fpt_sincos": [_vp, _vp, _i64, _int, _int, _vp],
    "fpt_sincos_f32": [_vp, _vp, _i64, _int, _int, _vp],
    "fpt_rope_table": [_vp, _vp, _i64, _i64, _int, _int, _vp],
    "fpt_rope_table_lut": [_vp, _vp, _vp, _i64, _i64, _int, _vp],
    "fpt_rope_apply": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _int, _vp],
    "fpt_attention_fwd": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                          ctypes.POINTER(_i64), ctypes.POINTER(_i64), _int, _int, ctypes.c_float, ctypes.c_float, _int, _vp, _vp],
    "fpt_attention_bwd_workspace_bytes": [_i64, _i64, _i64],
    "fpt_attention_bwd_fused_workspace_bytes": [_i64, _i64, _i64],
    "fpt_attention_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                          ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                          ctypes.POINTER(_i64), _int, _int, ctypes.c_float, ctypes.c_float, _int, _int, _vp, _vp],
    "fpt_attention_bwd_routed": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                 ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                                 ctypes.POINTER(_i64), _int, _int, ctypes.c_float, ctypes.c_float, _int, _int, _int, _int,
                                 _vp, _vp],
    "fpt_attention_fwd_routed": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, ctypes.POINTER(_i64),
                                 ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), _int, _int,
                                 ctypes.c_float, ctypes.c_float, _int, _int, _int, _vp, _vp],
    "fpt_selftest_umma": [_vp, _vp, _vp, _int, _vp, _vp],
    "fpt_selftest_bounded_wait": [_vp, _vp, _i64, _int, _vp],
    "fpt_rope_apply_static_table": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _int, _vp],
    "fpt_rope_static_table_capacity": [],
    "fpt_set_tuning": [ctypes.c_char_p, _int],
    "fpt_get_tuning": [ctypes.c_char_p, ctypes.POINTER(_int)],
}
_RESTYPES = {"fpt_status_string": ctypes.c_char_p, "fpt_version": ctypes.c_char_p,
             "fpt_rope_static_table_capacity": ctypes.c_int64, "fpt_attention_bwd_workspace_bytes": ctypes.c_int64,
             "fpt_attention_bwd_fused_workspace_bytes": ctypes.c_int64}
SIGNATURES["fpt_status_string"] = [_int]
SIGNATURES["fpt_version"] = []


class FptError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, function: str, status: int, message: str):
        super().__init__(f"{function} failed with status {status}: {message}")
        self.function, self.status = function, status


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raise ImportError (never fall back) if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with "
                "`python -m fast_polynomial_transcendentals_b200.build` (needs nvcc); "
                "this package has no CPU or PyTorch fallback")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, _int)
        _lib = lib
    return _lib


def check(function: str, status: int) -> None:
    if status != 0:
        raise FptError(function, status, load().fpt_status_string(status).decode())


def call(function: str, *args) -> None:
    check(function, getattr(load(), function)(*args))
