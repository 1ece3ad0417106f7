"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only the test-suite, the smoke check and the bench's CPU-baseline leg import
this module.  The shipped package never does: it talks to the CUDA library and
fails loudly when that is missing.

All 16-bit data are ``numpy.uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libfpt_oracle.so"

FP16, BF16 = 0, 1
CURRENT, SOLLYA = 0, 1
SHAPES = ("ODD_HALF", "ODD", "ODD_SAT", "SWISH", "XMUL_HALF", "EVEN", "ALG_SIG", "ALG_TANH")
SINCOS_VARIANTS = (
    "d3_d4_quarter_turn_fp16", "d3_d4_half_turn_fp16", "d5_d4_half_turn_fp16", "d5_d6_half_turn_fp16",
    "d7_d6_half_turn_fp16", "d3_d4_bf16", "d3_d4_quarter_turn_bf16", "d3_d4_half_turn_bf16",
    "d5_d6_half_turn_bf16", "d5_d4_half_turn_fp16_bf16",
)
ROPE_HALF_TURN_D5_D6, ROPE_QUARTER_TURN_D3_D4 = 0, 1

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i64 = ctypes.c_int64
_int = ctypes.c_int


def build(force: bool = False) -> Path:
    """Compile ``libfpt_oracle.so`` with the Makefile next to this file."""
    if force or not LIB_PATH.exists():
        subprocess.run(["make", "-C", str(HERE), "libfpt_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(LIB_PATH))
        L.fpt_oracle_find_program.argtypes = [ctypes.c_char_p, _int, _int]
        L.fpt_oracle_eval_lane.argtypes = [_int, ctypes.c_uint16]
        L.fpt_oracle_eval_lane.restype = ctypes.c_uint16
        L.fpt_oracle_program_info.argtypes = [_int, ctypes.c_char_p, _int, ctypes.POINTER(_int), ctypes.POINTER(_int),
                                              ctypes.POINTER(_int), ctypes.POINTER(_int), _u16p, _u16p]
        L.fpt_oracle_unary.argtypes = [_int, _u16p, _u16p, _i64]
        L.fpt_oracle_unary_repeat.argtypes = [_int, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_binary_bwd.argtypes = [_int, _u16p, _u16p, _u16p, _i64]
        L.fpt_oracle_swiglu.argtypes = [_int, _u16p, _u16p, _u16p, _i64]
        L.fpt_oracle_swiglu_packed.argtypes = [_int, _u16p, _u16p, _i64, _i64]
        L.fpt_oracle_swiglu_bwd.argtypes = [_int, _int, _u16p, _u16p, _u16p, _u16p, _u16p, _i64]
        L.fpt_oracle_swiglu_bwd_shared_sigmoid.argtypes = [_int, _u16p, _u16p, _u16p, _u16p, _u16p, _i64]
        L.fpt_oracle_b3_direct_bf16.argtypes = [_u16p, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_b3_direct_f32.argtypes = [_f32p, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_exp2_hinge.argtypes = [_u16p, _u16p, _i64, _int]
        L.fpt_oracle_exp2_hinge_repeat.argtypes = [_u16p, _u16p, _i64, _int, _int]
        L.fpt_oracle_multiply.argtypes = [_u16p, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_fma16.argtypes = [_u16p, _u16p, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_swish_shared_sigmoid.argtypes = [_u16p, _u16p, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_exp2_full_f32.argtypes = [_f32p, _f32p, _i64, _int]
        L.fpt_oracle_sincos_f32.argtypes = [_int, _f32p, _f32p, _i64, _int]
        L.fpt_oracle_sincos_f32.restype = ctypes.c_int
        L.fpt_oracle_sincos_packed.argtypes = [_int, _f32p, _u16p, _u16p, _i64]
        L.fpt_oracle_sincos_packed_compute.argtypes = [_int, _f32p, _u16p, _u16p, _i64, _int]
        L.fpt_oracle_rope_table.argtypes = [_int, _u32p, _u16p, _i64, _i64]
        L.fpt_oracle_rope_table_lut.argtypes = [_u32p, _u32p, _u16p, _i64, _i64, _int]
        L.fpt_oracle_rope_apply.argtypes = [_u16p, _u16p, _u32p, _u16p, _u16p, _i64, _i64, _i64, _i64, _i64, _int]
        L.fpt_oracle_attention_rows.argtypes = [_u16p, _u16p, _u16p, _f32p, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                                _i64p, _i64, _int, _int, ctypes.c_float, ctypes.c_float, _int]
        _lib = L
    return _lib


def _p16(a: np.ndarray):
    assert a.dtype == np.uint16 and a.flags.c_contiguous
    return a.ctypes.data_as(_u16p)


def _c16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


def set_threads(n: int = 0) -> int:
    """Use `n` OpenMP threads from now on (0: keep the current setting); returns the number in effect."""
    fn = lib().fpt_oracle_set_threads
    fn.argtypes = [ctypes.c_int]
    fn.restype = ctypes.c_int
    return int(fn(int(n)))


def find_program(name: str, dtype: int, source: int = CURRENT) -> int:
    idx = lib().fpt_oracle_find_program(name.encode(), dtype, source)
    if idx < 0:
        raise KeyError(f"no oracle program {name} dtype={dtype} source={source}")
    return idx


def program_table() -> list[dict]:
    L = lib()
    rows = []
    for i in range(L.fpt_oracle_program_count()):
        name = ctypes.create_string_buffer(32)
        dt, src, shape, deg = _int(), _int(), _int(), _int()
        clamp = ctypes.c_uint16()
        coeffs = (ctypes.c_uint16 * 7)()
        L.fpt_oracle_program_info(i, name, 32, dt, src, shape, deg, ctypes.byref(clamp), coeffs)
        rows.append(dict(name=name.value.decode(), dtype=dt.value, source=src.value, shape=SHAPES[shape.value],
                         degree=deg.value, clamp=clamp.value, coeffs=list(coeffs)))
    return rows


def eval_lane(program: int, x: int) -> int:
    return lib().fpt_oracle_eval_lane(program, x)


def unary(program: int, x: np.ndarray, repeats: int = 1) -> np.ndarray:
    x = _c16(x)
    out = np.empty_like(x)
    if repeats == 1:
        lib().fpt_oracle_unary(program, _p16(x), _p16(out), x.size)
    else:
        lib().fpt_oracle_unary_repeat(program, _p16(x), _p16(out), x.size, repeats)
    return out


def binary_bwd(program: int, grad_out: np.ndarray, x: np.ndarray) -> np.ndarray:
    go, x = _c16(grad_out), _c16(x)
    out = np.empty_like(x)
    lib().fpt_oracle_binary_bwd(program, _p16(go), _p16(x), _p16(out), x.size)
    return out


def swiglu(program: int, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate, up = _c16(gate), _c16(up)
    out = np.empty_like(gate)
    lib().fpt_oracle_swiglu(program, _p16(gate), _p16(up), _p16(out), gate.size)
    return out


def swiglu_packed(program: int, packed: np.ndarray) -> np.ndarray:
    packed = _c16(packed)
    rows, two_h = packed.shape
    out = np.empty((rows, two_h // 2), dtype=np.uint16)
    lib().fpt_oracle_swiglu_packed(program, _p16(packed), _p16(out), rows, two_h // 2)
    return out


def swiglu_bwd(fwd_program: int, bwd_program: int, grad_out, gate, up):
    go, gate, up = _c16(grad_out), _c16(gate), _c16(up)
    gg, gu = np.empty_like(gate), np.empty_like(gate)
    lib().fpt_oracle_swiglu_bwd(fwd_program, bwd_program, _p16(go), _p16(gate), _p16(up), _p16(gg), _p16(gu), gate.size)
    return gg, gu


def swiglu_bwd_shared_sigmoid(sigmoid_program: int, grad_out, gate, up):
    go, gate, up = _c16(grad_out), _c16(gate), _c16(up)
    gg, gu = np.empty_like(gate), np.empty_like(gate)
    lib().fpt_oracle_swiglu_bwd_shared_sigmoid(sigmoid_program, _p16(go), _p16(gate), _p16(up), _p16(gg), _p16(gu), gate.size)
    return gg, gu


def b3_direct(scores: np.ndarray, log2_n: int = 12, with_grad: bool = False):
    """scores: uint16 bf16 patterns, or float32 (rounded to bf16 first)."""
    scores = np.ascontiguousarray(scores)
    prob = np.empty(scores.shape, dtype=np.uint16)
    grad = np.empty(scores.shape, dtype=np.uint16) if with_grad else None
    gp = _p16(grad) if with_grad else None
    if scores.dtype == np.float32:
        lib().fpt_oracle_b3_direct_f32(scores.ctypes.data_as(_f32p), _p16(prob), gp, scores.size, log2_n)
    else:
        lib().fpt_oracle_b3_direct_bf16(_p16(_c16(scores)), _p16(prob), gp, scores.size, log2_n)
    return (prob, grad) if with_grad else prob


def multiply(a: np.ndarray, b: np.ndarray, dtype: int) -> np.ndarray:
    a, b = _c16(a), _c16(b)
    out = np.empty_like(a)
    lib().fpt_oracle_multiply(_p16(a), _p16(b), _p16(out), a.size, dtype)
    return out


def fma16(a: np.ndarray, b: np.ndarray, c: np.ndarray, dtype: int) -> np.ndarray:
    """One fused multiply-add per lane, a*b + c with a single rounding."""
    a, b, c = _c16(a), _c16(b), _c16(c)
    out = np.empty_like(a)
    lib().fpt_oracle_fma16(_p16(a), _p16(b), _p16(c), _p16(out), a.size, dtype)
    return out


def fwd_deriv(function: str, variant: str, x: np.ndarray):
    """(y, dy) of the FP16 forward-with-derivative composites; variant in {"alg", "poly", "shared"}."""
    x = _c16(x)
    if variant == "shared":
        s = unary(find_program("SIGMOID_FWD_D3", FP16), x)
        y, dy = np.empty_like(x), np.empty_like(x)
        lib().fpt_oracle_swish_shared_sigmoid(_p16(x), _p16(s), _p16(y), _p16(dy), x.size, FP16)
        return y, dy
    y = unary(find_program(f"{function}_FWD_D3", FP16), x)
    if variant == "alg":
        ones = np.full_like(x, 0x3c00)
        return y, binary_bwd(find_program(f"{function}_BWD_ALGEBRAIC", FP16), ones, y)
    ones = np.full_like(x, 0x3c00)
    return y, binary_bwd(find_program(f"{function}_BWD_D4", FP16), ones, x)


def fused_fwd_bwd(function: str, x: np.ndarray, grad_out: np.ndarray):
    """(y, grad_in) of the fused FP16 forward + gradient composites."""
    x, grad_out = _c16(x), _c16(grad_out)
    y = unary(find_program(f"{function}_FWD_D3", FP16), x)
    if function == "SWISH":
        return y, binary_bwd(find_program("SWISH_BWD_D4", FP16), grad_out, x)
    return y, binary_bwd(find_program(f"{function}_BWD_ALGEBRAIC", FP16), grad_out, y)


def exp2_hinge(x: np.ndarray, constant_set: int = 0, repeats: int = 1) -> np.ndarray:
    x = _c16(x)
    out = np.empty_like(x)
    if repeats == 1:
        lib().fpt_oracle_exp2_hinge(_p16(x), _p16(out), x.size, constant_set)
    else:
        lib().fpt_oracle_exp2_hinge_repeat(_p16(x), _p16(out), x.size, constant_set, repeats)
    return out


EXP2_FULL_D3, EXP2_FULL_PWL2, EXP2_FULL_D2_SAFE, EXP2_FULL_PWL2_SAFE_F16 = 0, 1, 2, 3


def exp2_full(x: np.ndarray, variant: int = EXP2_FULL_D3) -> np.ndarray:
    """fp32 2^x through the full-range software evaluators (bit pattern of the device functions)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().fpt_oracle_exp2_full_f32(x.ctypes.data_as(_f32p), out.ctypes.data_as(_f32p), x.size, variant)
    return out


SINCOS_F32_VARIANTS = ("native", "d3_d4", "d3_d4_cycle", "d3_d4_magic_bias", "d5_d4_half_turn_ls", "d5_d4_half_turn_sollya",
                       "d5_d4_half_turn_sollya_fast", "d5_d4", "d7_d6")


def sincos_f32(variant: str | int, angles: np.ndarray, iterations: int = 0) -> np.ndarray:
    """fp32 [2, n] (cos plane, sin plane) of one fp32 polynomial variant (1..8; the native control has no oracle)."""
    idx = SINCOS_F32_VARIANTS.index(variant) if isinstance(variant, str) else int(variant)
    angles = np.ascontiguousarray(angles, dtype=np.float32)
    out = np.empty((2, angles.size), dtype=np.float32)
    rc = lib().fpt_oracle_sincos_f32(idx, angles.ctypes.data_as(_f32p), out.ctypes.data_as(_f32p), angles.size, iterations)
    if rc != 0:
        raise ValueError(f"no fp32 sin/cos oracle for variant {variant!r}")
    return out


def sincos_packed(variant: str | int, angles: np.ndarray, iterations: int | None = None):
    """Returns (cos, sin) as uint16 patterns in the variant's output format."""
    v = SINCOS_VARIANTS.index(variant) if isinstance(variant, str) else variant
    angles = np.ascontiguousarray(angles, dtype=np.float32)
    c = np.empty(angles.shape, dtype=np.uint16)
    s = np.empty(angles.shape, dtype=np.uint16)
    if iterations is None:
        lib().fpt_oracle_sincos_packed(v, angles.ctypes.data_as(_f32p), _p16(c), _p16(s), angles.size)
    else:
        lib().fpt_oracle_sincos_packed_compute(v, angles.ctypes.data_as(_f32p), _p16(c), _p16(s), angles.size, iterations)
    return c, s


def rope_table(kind: int, increments: np.ndarray, seq: int) -> np.ndarray:
    inc = np.ascontiguousarray(increments).view(np.uint32)
    table = np.empty((2, seq, inc.size), dtype=np.uint16)
    lib().fpt_oracle_rope_table(kind, inc.ctypes.data_as(_u32p), _p16(table), seq, inc.size)
    return table


def rope_phase_table() -> np.ndarray:
    """The [128, 2] fp16 table the look-up variant expects: (sin, cos) of 2*pi*i/128, as uint16 bit patterns."""
    t = 2.0 * np.pi * np.arange(128) / 128.0
    return np.stack([np.sin(t), np.cos(t)], axis=1).astype(np.float16).view(np.uint16)


def rope_table_lut(increments: np.ndarray, phase_table: np.ndarray, seq: int, iterations: int = 0) -> np.ndarray:
    inc = np.ascontiguousarray(increments).view(np.uint32)
    lut = np.ascontiguousarray(phase_table, dtype=np.uint16).reshape(128, 2).view(np.uint32).reshape(128)
    table = np.empty((2, seq, inc.size), dtype=np.uint16)
    lib().fpt_oracle_rope_table_lut(inc.ctypes.data_as(_u32p), lut.ctypes.data_as(_u32p), _p16(table), seq, inc.size,
                                    iterations)
    return table


def rope_apply(q: np.ndarray, k: np.ndarray, increments: np.ndarray, io_bf16: bool = False):
    """q [B,S,Hq,D], k [B,S,Hk,D] -> transposed [B,H,S,D]; one increment per (even, odd) pair."""
    q, k = _c16(q), _c16(k)
    inc = np.ascontiguousarray(increments).view(np.uint32)
    B, S, Hq, D = q.shape
    Hk = k.shape[2]
    assert inc.size == D // 2
    qo = np.empty((B, Hq, S, D), dtype=np.uint16)
    ko = np.empty((B, Hk, S, D), dtype=np.uint16)
    lib().fpt_oracle_rope_apply(_p16(q), _p16(k), inc.ctypes.data_as(_u32p), _p16(qo), _p16(ko), B, S, Hq, Hk, D, int(io_bf16))
    return qo, ko


ATTN_SOFTCAP_TANH, ATTN_SIGMOID_B3, ATTN_SOFTMAX, ATTN_SOFTCAP_NATIVE, ATTN_SIGMOID_NATIVE = 0, 1, 2, 3, 4


def attention_rows(q, k, v, b: int, hq: int, rows, mode: int, causal: bool, scale: float,
                   softcap: float = 0.0, log2_n: int = 12) -> np.ndarray:
    """fp32 attention of selected query rows; q,k,v are (B,S,H,D) bf16 patterns."""
    q, k, v = _c16(q), _c16(k), _c16(v)
    B, S, Hq, D = q.shape
    Hk = k.shape[2]
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    out = np.empty((rows.size, D), dtype=np.float32)
    lib().fpt_oracle_attention_rows(_p16(q), _p16(k), _p16(v), out.ctypes.data_as(_f32p), B, S, Hq, Hk, D, b, hq,
                                    rows.ctypes.data_as(_i64p), rows.size, mode, int(causal), scale, softcap, log2_n)
    return out


# ---- bit-pattern helpers shared by tests ------------------------------------

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 patterns (NaN -> 0x7fff like cvt.rn.bf16.f32)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    r[nan] = 0x7FFF
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float16).view(np.uint16)


def f16_from_bits(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b, dtype=np.uint16).view(np.float16)
