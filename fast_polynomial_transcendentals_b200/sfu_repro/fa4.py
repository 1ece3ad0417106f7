"""Declarative attention configuration and the PyTorch wrapper, bound to this package's attention kernel.

Keeps the reference's configuration surface (reference: src/sfu_repro/fa4.py:50-103 the two dataclasses, :106-199
exp2 routing variants, :271-415 validation, :454-647 resolution against a runtime mapping, :650-752 the canonical B2 /
B3 / B5 configurations, :755-948 autograd function and module wrapper): same field names, defaults, accepted values
and error messages, and the same seam -- ``resolve_fa4_config(config, runtime=...)`` takes a mapping with the keys
``flash_attn_fwd``, ``flash_attn_bwd``, ``run_polynomial_coefficient_audit``, ``audit_polynomial_selection``,
``audit_attention_handwritten_fast_path``, ``create_softcap_scoremod_backend``,
``create_softcap_scoremod_bwd_backend``.  When no mapping is passed, the runtime is this package's own
(``b200_runtime()``): forward and backward on the tcgen05 kernels of this package.

Inputs of :class:`FA4AttentionWrapper` are ``(batch, heads, sequence, dim)``; the kernel interface is
``(batch, sequence, heads, dim)``.
"""
from __future__ import annotations

import logging
import math
import os
from collections.abc import Callable, Mapping
from dataclasses import dataclass
from functools import lru_cache
from typing import Any

import torch
from torch import nn

LOGGER = logging.getLogger(__name__)

FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH = 4096

SUPPORTED_EXP2_BACKENDS = ("d3", "pwl2", "pwl1_safe", "pwl1_safe_f16", "pwl2_safe", "pwl2_safe_f16", "pwl2_safe_bf16",
                           "d2_safe", "d2_safe_noclamp", "d2_safe_f16", "d2_safe_bf16", "pwl2_f16")


@dataclass(frozen=True)
class FA4Config:
    """What the user asks for; independent of any training framework."""

    mode: str = "softmax"
    exp2_emu_backend: str = "d3"
    exp2_emu_freq: int | None = None
    exp2_emu_freq_bwd: int = 0
    softcap: float = 30.0
    softcap_backend: str = "native"
    softcap_degree: int = 4
    softcap_coeff_source: str = "current"
    softcap_backward_mode: str = "analytical"
    sigmoid_variant: str = "poly"
    sigmoid_poly_backend: str = "cute"
    sigmoid_degree: int = 3
    sigmoid_degree_bwd: int | None = None
    sigmoid_coeff_source: str = "current"
    sigmoid_backward_mode: str = "algebraic"
    sigmoid_sfu_freq: int = 16
    sigmoid_sfu_res: int = 0
    sigmoid_sfu_freq_bwd: int | None = None
    sigmoid_sfu_res_bwd: int | None = None
    sigmoid_bias: float | None = None
    sigmoid_qk_norm: bool = True
    audit_coefficients: bool = True


@dataclass(frozen=True)
class ResolvedFA4Config:
    """A validated configuration bound to an attention runtime."""

    mode: str
    flash_attn_fwd: Callable[..., Any]
    flash_attn_bwd: Callable[..., Any]
    exp2_emu_backend: str = "d3"
    exp2_emu_freq: int | None = None
    exp2_emu_freq_bwd: int = 0
    softcap: float = 0.0
    score_mod: Callable[..., Any] | None = None
    score_mod_bwd: Callable[..., Any] | None = None
    sigmoid_attention: bool = False
    sigmoid_sfu_freq: int = 16
    sigmoid_sfu_res: int = 0
    sigmoid_sfu_freq_bwd: int | None = None
    sigmoid_sfu_res_bwd: int | None = None
    sigmoid_use_direct_bwd_poly: bool = False
    sigmoid_bias: float | None = None
    sigmoid_poly_backend: str = "cute"
    sigmoid_degree: int = 3
    sigmoid_degree_bwd: int | None = None
    sigmoid_coeff_source: str = "current"
    sigmoid_qk_norm: bool = True
    implementation_summary: str = ""


@dataclass(frozen=True)
class Exp2Variant:
    """One mixed SFU / software exp2 route of the softmax benchmark."""

    name: str
    backend: str
    forward_frequency: int | None
    backward_frequency: int

    @staticmethod
    def _fraction(frequency: int | None) -> float | None:
        if frequency is None:
            return None
        return 0.0 if frequency == 0 else min(1.0, 4.0 / frequency)

    @property
    def nominal_forward_polynomial_fraction(self) -> float | None:
        return self._fraction(self.forward_frequency)

    @property
    def nominal_backward_polynomial_fraction(self) -> float:
        return float(self._fraction(self.backward_frequency))

    @property
    def nominal_forward_pwl_fraction(self) -> float | None:
        return self.nominal_forward_polynomial_fraction

    @property
    def nominal_backward_pwl_fraction(self) -> float:
        return self.nominal_backward_polynomial_fraction


DEFAULT_EXP2_VARIANTS = ",".join(("sfu=d3:0:0", "d3_auto=d3:auto:0", "d2_safe_12p5=d2_safe:32:0", "d2_safe_16p7=d2_safe:24:0",
                                  "d2_safe_20=d2_safe:20:0", "d2_safe_25=d2_safe:16:0", "d2_safe_33p3=d2_safe:12:0",
                                  "d2_safe_40=d2_safe:10:0", "d2_safe_50=d2_safe:8:0", "d2_safe_66p7=d2_safe:6:0",
                                  "d2_safe_100=d2_safe:4:0"))


def _validate_exp2_route(frequency: int | None, label: str) -> int | None:
    if frequency is None:
        return None
    frequency = int(frequency)
    if frequency < 0 or (frequency != 0 and (frequency < 4 or frequency % 2)):
        raise ValueError(f"{label} frequency must be 0 or an even integer >= 4, got {frequency}")
    return frequency


def parse_exp2_frequency(value: str, *, allow_auto: bool) -> int | None:
    """One exp2 routing frequency: 'auto' (where allowed), 0, or an even integer >= 4."""
    if allow_auto and value == "auto":
        return None
    try:
        frequency = int(value)
    except ValueError as error:
        allowed = "'auto', 0, or an even integer >= 4" if allow_auto else "0 or an even integer >= 4"
        raise ValueError(f"frequency must be {allowed}, got {value!r}") from error
    return _validate_exp2_route(frequency, "exp2")


def parse_exp2_variants(value: str) -> tuple[Exp2Variant, ...]:
    """Parse ``name=backend:forward:backward`` items separated by commas."""
    variants: list[Exp2Variant] = []
    for raw in (item.strip() for item in value.split(",")):
        if not raw:
            continue
        try:
            name, route = raw.split("=", maxsplit=1)
            backend, forward, backward = route.split(":")
        except ValueError as error:
            raise ValueError("variant must have name=backend:forward_frequency:backward_frequency syntax, "
                             f"got {raw!r}") from error
        name, backend = name.strip(), backend.strip()
        if not name:
            raise ValueError("variant name must not be empty")
        if backend not in SUPPORTED_EXP2_BACKENDS:
            raise ValueError(f"unsupported exp2 backend {backend!r}")
        variants.append(Exp2Variant(name, backend, parse_exp2_frequency(forward.strip(), allow_auto=True),
                                    int(parse_exp2_frequency(backward.strip(), allow_auto=False))))
    if not variants:
        raise ValueError("at least one variant is required")
    if len({v.name for v in variants}) != len(variants):
        raise ValueError("variant names must be unique")
    return tuple(variants)


def _env_flag(name: str) -> bool:
    value = os.environ.get(name)
    return value is not None and value.lower() in ("1", "true", "yes", "on")


def _sigmoid_route(frequency: int, residue_count: int, label: str) -> tuple[int, int]:
    frequency, residue_count = int(frequency), int(residue_count)
    if frequency <= 0:
        raise ValueError(f"{label} sigmoid_sfu_freq must be positive, got {frequency}")
    if residue_count < 0 or residue_count > frequency:
        raise ValueError(f"{label} sigmoid_sfu_res must lie in [0, sigmoid_sfu_freq], got {residue_count} for {frequency}")
    return frequency, residue_count


def _uses_sollya(c: FA4Config) -> bool:
    return (c.mode == "softcap" and c.softcap_coeff_source == "sollya") or (
        c.mode == "sigmoid_attention" and c.sigmoid_variant == "poly" and c.sigmoid_coeff_source == "sollya")


def _is_device_current_poly(c: FA4Config, degree: int) -> bool:
    return (c.mode == "sigmoid_attention" and c.sigmoid_variant == "poly" and c.sigmoid_poly_backend == "device"
            and c.sigmoid_coeff_source == "current" and int(c.sigmoid_degree) == degree and c.sigmoid_bias is None)


def _uses_direct_flash_sigmoid(c: FA4Config) -> bool:
    return _is_device_current_poly(c, 3)


def _check_choice(value, allowed, message):
    if value not in allowed:
        raise ValueError(message)


def validate_fa4_config(config: FA4Config, *, sequence_length: int | None = None) -> FA4Config:
    """Check a configuration without touching CUDA or any attention backend."""
    c = config
    _check_choice(c.mode, ("softmax", "softcap", "sigmoid_attention"), f"unsupported FA4 mode {c.mode!r}")
    _check_choice(c.exp2_emu_backend, SUPPORTED_EXP2_BACKENDS, f"unsupported exp2 backend {c.exp2_emu_backend!r}")
    _validate_exp2_route(c.exp2_emu_freq, "forward exp2")
    _validate_exp2_route(c.exp2_emu_freq_bwd, "backward exp2")
    if _uses_sollya(c) and not _env_flag("SFU_REPRO_ALLOW_SOLLYA_SWEEP"):
        raise ValueError("Sollya coefficient sources are benchmark-only. Set SFU_REPRO_ALLOW_SOLLYA_SWEEP=1 for an "
                         "explicit sweep.")

    if c.mode == "softcap":
        _check_choice(c.softcap_backend, ("native", "cute", "device"), f"unsupported softcap backend {c.softcap_backend!r}")
        _check_choice(c.softcap_backward_mode, ("analytical", "ste", "exact_1mt2", "native"),
                      f"unsupported softcap backward mode {c.softcap_backward_mode!r}")
        _check_choice(c.softcap_coeff_source, ("current", "sollya"),
                      f"unsupported softcap coefficient source {c.softcap_coeff_source!r}")
        if c.softcap <= 0:
            raise ValueError("softcap must be positive")
        native = c.softcap_backend == "native"
        if native and c.softcap_backward_mode != "native":
            raise ValueError("native softcap requires softcap_backward_mode='native'")
        if not native and c.softcap_backward_mode == "native":
            raise ValueError("polynomial softcap cannot use softcap_backward_mode='native'")
        if c.softcap_coeff_source == "sollya" and c.softcap_backend != "device":
            raise ValueError("Sollya softcap fits require softcap_backend='device'")

    if c.mode == "sigmoid_attention":
        _check_choice(c.sigmoid_variant, ("poly", "sfu"), f"unsupported sigmoid variant {c.sigmoid_variant!r}")
        _check_choice(c.sigmoid_poly_backend, ("cute", "device"),
                      f"unsupported sigmoid polynomial backend {c.sigmoid_poly_backend!r}")
        _check_choice(c.sigmoid_backward_mode, ("algebraic", "direct"),
                      f"unsupported sigmoid backward mode {c.sigmoid_backward_mode!r}")
        _check_choice(c.sigmoid_coeff_source, ("current", "sollya"),
                      f"unsupported sigmoid coefficient source {c.sigmoid_coeff_source!r}")
        if int(c.sigmoid_degree) not in (2, 3, 4, 5, 6):
            raise ValueError("sigmoid_degree must be one of 2, 3, 4, 5, or 6")
        if c.sigmoid_degree_bwd is not None and int(c.sigmoid_degree_bwd) not in (2, 3, 4, 5, 6):
            raise ValueError("sigmoid_degree_bwd must be one of 2, 3, 4, 5, or 6")
        poly = c.sigmoid_variant == "poly"
        if poly and c.sigmoid_poly_backend == "cute":
            raise ValueError("causal polynomial sigmoid attention requires sigmoid_poly_backend='device'")
        if poly and c.sigmoid_coeff_source == "sollya" and c.sigmoid_poly_backend != "device":
            raise ValueError("Sollya sigmoid fits require sigmoid_poly_backend='device'")
        fwd_freq, fwd_res = _sigmoid_route(c.sigmoid_sfu_freq, c.sigmoid_sfu_res, "forward")
        bwd_freq, bwd_res = _sigmoid_route(fwd_freq if c.sigmoid_sfu_freq_bwd is None else c.sigmoid_sfu_freq_bwd,
                                           fwd_res if c.sigmoid_sfu_res_bwd is None else c.sigmoid_sfu_res_bwd, "backward")
        if poly and (fwd_res != 0 or bwd_res != 0):
            raise ValueError("sigmoid_variant='poly' must route every forward/backward lane through the polynomial")
        if not poly and (fwd_res != fwd_freq or bwd_res != bwd_freq):
            raise ValueError("sigmoid_variant='sfu' must route every forward/backward lane through the SFU")
        if _is_device_current_poly(c, 2) and c.sigmoid_backward_mode != "algebraic":
            raise ValueError("bias-aware FlashSigmoid D2 requires sigmoid_backward_mode='algebraic'")
        if _uses_direct_flash_sigmoid(c):
            if sequence_length is None:
                raise ValueError("direct FlashSigmoid D3 requires an explicit sequence_length")
            if int(sequence_length) != FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH:
                raise ValueError("direct FlashSigmoid D3/D4 is fitted for sequence length "
                                 f"{FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH}, got {sequence_length}")
    return config


# ---- this package's attention runtime ----------------------------------------------------------------

# exp2 backends built into this package's attention kernels -> FPT_EXP2_FULL_* of the C ABI
_EXP2_BACKEND_IDS = {"d3": 0, "pwl2": 1, "d2_safe": 2, "pwl2_safe_f16": 3}
_BUILT_EXP2_FREQUENCIES = (0, 8, 12, 16, 32)


@dataclass(frozen=True)
class SoftcapScoreMod:
    """Token for `score_mod=`: soft-cap through the packed bf16 tanh polynomial inside the attention kernel."""

    softcap: float
    degree: int = 4
    backend: str = "device"
    coeff_source: str = "current"
    backward_mode: str = "analytical"


def _exp2_route(mode: int, backend: str, frequency, where: str) -> int:
    """Validated routing frequency for the kernels; None ('automatic') keeps every lane on the SFU here."""
    route = 0 if frequency is None else int(frequency)
    if route == 0:
        return 0
    if mode != 2:
        raise NotImplementedError(f"{where}: software exp2 routing is built for the plain soft-max only"
                                  + ("" if mode != 0 or where != "forward" else " (and the cubic 'd3' under a soft-cap)"))
    if backend not in _EXP2_BACKEND_IDS:
        raise NotImplementedError(f"{where}: exp2 backend {backend!r} is not built; built: "
                                  + ", ".join(repr(b) for b in _EXP2_BACKEND_IDS))
    if route not in _BUILT_EXP2_FREQUENCIES:
        raise NotImplementedError(f"{where}: built routing frequencies are {_BUILT_EXP2_FREQUENCIES}, got {route}")
    return route


def _sigmoid_mode(seq: int, *, sigmoid_sfu_freq, sigmoid_sfu_res, sigmoid_bias, polynomial_ok: bool, what: str):
    """(kernel mode, log2_n) of a sigmoid-attention call: the direct cubic (every lane polynomial) or its native twin
    (every lane on the SFU).  Both take the bias -log(n) for a power of two n (default n = sequence length)."""
    if sigmoid_bias is None:
        if seq & (seq - 1):
            raise NotImplementedError("sigmoid attention needs a power-of-two sequence length (bias -log n)")
        log2_n = seq.bit_length() - 1
    else:
        log2_n = round(-float(sigmoid_bias) / math.log(2.0))
        if log2_n < 1 or log2_n > 24 or abs(-log2_n * math.log(2.0) - float(sigmoid_bias)) > 1e-6:
            raise NotImplementedError("sigmoid_bias must be -log(n) for a power of two n in [2, 2^24]")
    all_poly, all_sfu = int(sigmoid_sfu_res) == 0, int(sigmoid_sfu_res) == int(sigmoid_sfu_freq)
    if all_sfu:
        return 4, log2_n
    if not (all_poly and polynomial_ok and sigmoid_bias is None):
        raise NotImplementedError(what)
    return 1, log2_n


class _AttentionStatus:
    """The status word the attention kernels report bounded-wait timeouts through, one per device.

    The word lives on the device for the life of the process (no allocation or memset per call).  After every launch
    its value is copied to pinned host memory on the launching stream; `poll` reads that copy once the copy has
    completed (never blocking), `check` waits for it.  A non-zero word means a device-side wait ran out and the outputs
    of the call that set it (and of every later call: blocks that find the word set do no work) are invalid.  The word
    is cleared when the error is raised, so the call after the exception runs normally."""

    def __init__(self, device):
        self.device = device
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.where = ""

    def after_launch(self, where: str) -> None:
        if torch.cuda.is_current_stream_capturing():     # a captured launch is checked when the caller asks (check())
            return
        self.host.copy_(self.word, non_blocking=True)
        self.event.record(torch.cuda.current_stream(self.device))
        self.pending, self.where = True, where

    def _raise_if_set(self) -> None:
        self.pending = False
        value = int(self.host.item()) & 0xFFFFFFFF
        if value:
            from .. import _lib
            self.word.zero_()
            self.host.zero_()
            message = _lib.load().fpt_status_string(-8).decode()      # FPT_ERR_DEVICE_TIMEOUT
            raise RuntimeError(f"{message}: status word {value:#010x} (waiting point {value & 0xFFFF}) seen after "
                               f"{self.where}; the outputs of that call are invalid")

    def poll(self) -> None:
        if self.pending and not torch.cuda.is_current_stream_capturing() and self.event.query():
            self._raise_if_set()

    def check(self) -> None:
        if not self.pending:             # nothing copied yet (captured launches): read the word itself
            self.host.copy_(self.word)
            self.where = self.where or "an attention launch"
        else:
            self.event.synchronize()
        self._raise_if_set()


_STATUS: dict[Any, _AttentionStatus] = {}


def _status_for(device) -> _AttentionStatus:
    key = torch.device(device)
    key = torch.device("cuda", torch.cuda.current_device()) if key.index is None else key
    state = _STATUS.get(key)
    if state is None:
        state = _STATUS[key] = _AttentionStatus(key)
    return state


def check_attention_status(device=None) -> None:
    """Wait for the attention launches enqueued so far on `device` (default: every device used) and raise RuntimeError
    if one of them reported a device-side timeout.  Without this call the same error surfaces, without blocking, at the
    first attention call made after the failed launch has finished; FPT_CHECK_STATUS=1 checks after every call."""
    for state in ([_status_for(device)] if device is not None else list(_STATUS.values())):
        state.check()


def _finish_launch(state: _AttentionStatus, where: str) -> None:
    state.after_launch(where)
    if _env_flag("FPT_CHECK_STATUS"):
        state.check()


def _b200_flash_attn_fwd(q, k, v, *, softmax_scale=None, causal=True, softcap=0.0, score_mod=None, sigmoid_attention=False,
                         sigmoid_sfu_freq=16, sigmoid_sfu_res=0, sigmoid_bias=None, sigmoid_poly_backend="device",
                         sigmoid_degree=3, sigmoid_coeff_source="current", exp2_emu_backend="d3", exp2_emu_freq=None):
    """(out, lse) for (batch, seq, heads, dim) bf16 tensors on the tcgen05 kernel of this package."""
    import ctypes

    from .. import _lib
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise RuntimeError("the B200 attention kernel takes bfloat16 q, k, v")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("q, k, v must be CUDA tensors")
    if q.stride(-1) != 1 or k.stride(-1) != 1 or v.stride(-1) != 1:
        raise RuntimeError("the head dimension must be contiguous")
    batch, seq, q_heads, dim = q.shape
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(dim)
    log2_n = 12
    if sigmoid_attention:
        mode, log2_n = _sigmoid_mode(
            seq, sigmoid_sfu_freq=sigmoid_sfu_freq, sigmoid_sfu_res=sigmoid_sfu_res, sigmoid_bias=sigmoid_bias,
            polynomial_ok=(sigmoid_poly_backend == "device" and int(sigmoid_degree) == 3 and sigmoid_coeff_source == "current"),
            what="built sigmoid routes: the direct piecewise cubic on every lane (device, degree 3, current "
                 "coefficients, bias -log n) and the SFU sigmoid on every lane")
        cap = 0.0
    elif score_mod is not None:
        if not isinstance(score_mod, SoftcapScoreMod) or score_mod.degree != 4 or score_mod.coeff_source != "current":
            raise NotImplementedError("only the degree-4 'current' tanh soft-cap score-mod is built")
        mode, cap = 0, float(score_mod.softcap)
    elif softcap and float(softcap) > 0.0:
        mode, cap = 3, float(softcap)          # native twin: tanh on the special-function unit
    else:
        mode, cap = 2, 0.0
    if mode == 0 and exp2_emu_freq not in (None, 0) and exp2_emu_backend == "d3" and int(exp2_emu_freq) in _BUILT_EXP2_FREQUENCIES:
        route = int(exp2_emu_freq)             # the cubic is also routed under the polynomial soft-cap
    else:
        route = _exp2_route(mode, exp2_emu_backend, exp2_emu_freq, "forward")
    out = torch.empty((batch, seq, q_heads, dim), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((batch, q_heads, seq), dtype=torch.float32, device=q.device)
    strides = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    with torch.cuda.device(q.device):
        status = _status_for(q.device)
        status.poll()
        _lib.call("fpt_attention_fwd_routed", out.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), batch,
                  seq, q_heads, k.shape[2], dim, strides(q), strides(k), strides(v), strides(out), mode, int(bool(causal)),
                  scale, cap, log2_n, _EXP2_BACKEND_IDS.get(exp2_emu_backend, 0), route, status.word.data_ptr(),
                  torch.cuda.current_stream(q.device).cuda_stream)
        _finish_launch(status, "the attention forward")
    return out, lse


def _b200_flash_attn_bwd(q, k, v, out, dout, lse, softmax_scale=None, causal=True, softcap=0.0, *, score_mod=None,
                         score_mod_bwd=None, sigmoid_attention=False, sigmoid_bias=None, sigmoid_sfu_freq=16,
                         sigmoid_sfu_res=0, sigmoid_use_direct_bwd_poly=True, sigmoid_poly_backend="device",
                         sigmoid_degree=3, sigmoid_gradient_degree=4, sigmoid_coeff_source="current",
                         exp2_emu_backend="d3", exp2_emu_freq=0):
    """(dq, dk, dv) for the forward above (reference contract: src/sfu_repro/fa4.py:828-859)."""
    import ctypes

    from .. import _lib
    for name, t in (("q", q), ("k", k), ("v", v), ("dout", dout)):
        if t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(-1) != 1:
            raise RuntimeError(f"{name} must be a bfloat16 CUDA tensor with a contiguous head dimension")
    batch, seq, q_heads, dim = q.shape
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(dim)
    log2_n, grad_mode = 12, 0
    if sigmoid_attention:
        mode, log2_n = _sigmoid_mode(
            seq, sigmoid_sfu_freq=sigmoid_sfu_freq, sigmoid_sfu_res=sigmoid_sfu_res, sigmoid_bias=sigmoid_bias,
            polynomial_ok=(sigmoid_use_direct_bwd_poly and sigmoid_poly_backend == "device" and int(sigmoid_degree) == 3
                           and int(sigmoid_gradient_degree) == 4 and sigmoid_coeff_source == "current"),
            what="built sigmoid backward routes: the direct cubic with its coupled degree-4 derivative on every lane "
                 "(device, current coefficients, bias -log n) and the SFU sigmoid with p(1-p) on every lane")
        cap = 0.0
    elif score_mod is not None or score_mod_bwd is not None:
        token = score_mod_bwd if score_mod_bwd is not None else score_mod
        if not isinstance(token, SoftcapScoreMod) or token.degree != 4 or token.coeff_source != "current":
            raise NotImplementedError("only the degree-4 'current' tanh soft-cap score-mod is built")
        if token.backward_mode not in ("analytical", "exact_1mt2"):
            raise NotImplementedError(f"soft-cap backward mode {token.backward_mode!r} is not built "
                                      "(built: 'analytical', 'exact_1mt2')")
        mode, cap, grad_mode = 0, float(token.softcap), (0 if token.backward_mode == "analytical" else 1)
    elif softcap and float(softcap) > 0.0:
        mode, cap, grad_mode = 3, float(softcap), 1      # native twin: SFU tanh, derivative 1 - t^2
    else:
        mode, cap = 2, 0.0
    route = _exp2_route(mode, exp2_emu_backend, exp2_emu_freq, "backward")
    dq = torch.empty((batch, seq, q_heads, dim), dtype=torch.bfloat16, device=q.device)
    dk = torch.empty((batch, seq, k.shape[2], dim), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty_like(dk)
    strides = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    needs_forward = mode not in (1, 4)
    if needs_forward and (out is None or lse is None):
        raise RuntimeError("soft-max attention backward needs the forward's out and lse")
    # The single-pass form by default (5 matrix products, fp32 dQ buffer in the workspace; it accumulates dQ with additions
    # whose order is not fixed, so the last bit of dQ is not reproducible from run to run).
    # FPT_ATTENTION_BWD_SINGLE_PASS=0 asks for the deterministic two-pass form: the smaller workspace selects it.
    if os.environ.get("FPT_ATTENTION_BWD_SINGLE_PASS", "1").strip().lower() not in ("0", "false", "no", "off"):
        need = int(_lib.load().fpt_attention_bwd_fused_workspace_bytes(batch, seq, q_heads))
    else:
        need = int(_lib.load().fpt_attention_bwd_workspace_bytes(batch, seq, q_heads)) if needs_forward else 0
    workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        status = _status_for(q.device)
        status.poll()
        _lib.call("fpt_attention_bwd_routed", dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(),
                  k.data_ptr(), v.data_ptr(), out.data_ptr() if needs_forward else None,
                  lse.data_ptr() if needs_forward else None, workspace.data_ptr(), need, batch, seq, q_heads, k.shape[2],
                  dim, strides(q), strides(k), strides(v), strides(out) if needs_forward else strides(q), strides(dout),
                  mode, int(bool(causal)), scale, cap, log2_n, grad_mode, _EXP2_BACKEND_IDS.get(exp2_emu_backend, 0), route,
                  status.word.data_ptr(),
                  torch.cuda.current_stream(q.device).cuda_stream)
        _finish_launch(status, "the attention backward")
    return dq, dk, dv


@lru_cache(maxsize=1)
def b200_runtime() -> Mapping[str, Any]:
    """The runtime mapping `resolve_fa4_config` binds by default: this package's kernel and its own audits."""
    from .. import _lib
    _lib.load()

    def run_polynomial_coefficient_audit():
        # the constants compiled into the library are the ones pinned by tests/golden/program_table.json
        return [f"program_table[{_lib.load().fpt_program_count()}]"]

    def audit_polynomial_selection(selections):
        names = []
        for family, degree, source in selections:
            ok = (family, int(degree), source) in (("tanh_fwd", 4, "current"), ("sigmoid_fwd", 3, "current"),
                                                   ("sigmoid_bwd", 4, "current"))
            if not ok:
                raise RuntimeError(f"no audited attention polynomial for {family} degree {degree} source {source}")
            names.append(f"{family}_d{degree}_{source}")
        return names

    def audit_attention_handwritten_fast_path(family, degree, source):
        audit_polynomial_selection((({"flash_sigmoid_direct": "sigmoid_fwd", "flash_sigmoid_direct_with_grad": "sigmoid_bwd",
                                      "tanh_grad_analytical": "tanh_fwd"}.get(family, family), degree, source),))
        return f"B200 packed bf16 {family} D{int(degree)} {source}"

    def create_softcap_scoremod_backend(softcap, *, degree, backend, coeff_source):
        return SoftcapScoreMod(float(softcap), int(degree), backend, coeff_source)

    def create_softcap_scoremod_bwd_backend(softcap, *, degree, backend, backward_mode, coeff_source):
        return SoftcapScoreMod(float(softcap), int(degree), backend, coeff_source, backward_mode)

    return {"flash_attn_fwd": _b200_flash_attn_fwd, "flash_attn_bwd": _b200_flash_attn_bwd,
            "run_polynomial_coefficient_audit": run_polynomial_coefficient_audit,
            "audit_polynomial_selection": audit_polynomial_selection,
            "audit_attention_handwritten_fast_path": audit_attention_handwritten_fast_path,
            "create_softcap_scoremod_backend": create_softcap_scoremod_backend,
            "create_softcap_scoremod_bwd_backend": create_softcap_scoremod_bwd_backend}


def _load_fa4_runtime() -> Mapping[str, Any]:
    try:
        return b200_runtime()
    except (ImportError, OSError) as error:
        raise RuntimeError("The attention runtime is unavailable: build the kernel library with "
                           "`python -m fast_polynomial_transcendentals_b200.build`.") from error


def _require_built(c: FA4Config) -> None:
    """Reject, at resolution time, what this package's kernels do not run (a foreign runtime decides for itself)."""
    def refuse(what: str):
        raise NotImplementedError(
            f"{what} is not built in this package's attention kernels.  Built: soft-max with exp2 backends "
            f"{', '.join(_EXP2_BACKEND_IDS)} at routing frequencies {_BUILT_EXP2_FREQUENCIES} forward and backward "
            "('automatic' keeps every lane on the SFU); soft-cap native (SFU tanh) or polynomial degree 4 'current' "
            "with backward 'analytical' / 'exact_1mt2'; sigmoid attention 'sfu' or the direct D3 / coupled D4 "
            "polynomial pair with bias -log n")
    if c.mode == "softmax":
        routes = [f for f in (c.exp2_emu_freq, c.exp2_emu_freq_bwd) if f not in (None, 0)]
        if routes and c.exp2_emu_backend not in _EXP2_BACKEND_IDS:
            refuse(f"exp2 backend {c.exp2_emu_backend!r}")
        for f in routes:
            if int(f) not in _BUILT_EXP2_FREQUENCIES:
                refuse(f"exp2 routing frequency {f}")
    elif c.mode == "softcap" and c.softcap_backend != "native":
        if int(c.softcap_degree) != 4 or c.softcap_coeff_source != "current":
            refuse(f"soft-cap polynomial degree {c.softcap_degree} source {c.softcap_coeff_source!r}")
        if c.softcap_backward_mode not in ("analytical", "exact_1mt2"):
            refuse(f"soft-cap backward mode {c.softcap_backward_mode!r}")
    elif c.mode == "sigmoid_attention":
        if c.sigmoid_variant == "sfu":
            if c.sigmoid_bias is not None:
                k = round(-float(c.sigmoid_bias) / math.log(2.0))
                if k < 1 or k > 24 or abs(-k * math.log(2.0) - float(c.sigmoid_bias)) > 1e-6:
                    refuse(f"sigmoid_bias {c.sigmoid_bias} (not -log of a power of two)")
        elif not (_uses_direct_flash_sigmoid(c) and c.sigmoid_backward_mode == "direct"
                  and (c.sigmoid_degree_bwd is None or int(c.sigmoid_degree_bwd) == 4)):
            refuse("this polynomial sigmoid selection")


def resolve_fa4_config(config: FA4Config, *, sequence_length: int | None = None,
                       runtime: Mapping[str, Any] | None = None) -> ResolvedFA4Config:
    """Validate `config` and bind it to an attention runtime (this package's unless `runtime` is given)."""
    validate_fa4_config(config, sequence_length=sequence_length)
    own_runtime = runtime is None
    if own_runtime:
        _require_built(config)
    runtime = _load_fa4_runtime() if runtime is None else runtime
    c = config
    fwd, bwd = runtime["flash_attn_fwd"], runtime["flash_attn_bwd"]
    degree = int(c.sigmoid_degree)
    degree_bwd = degree if c.sigmoid_degree_bwd is None else int(c.sigmoid_degree_bwd)
    bias_aware_d2 = _is_device_current_poly(c, 2)
    direct = _uses_direct_flash_sigmoid(c)

    if c.audit_coefficients:
        audited = list(runtime["run_polynomial_coefficient_audit"]())
        selections: list[tuple[str, int, str]] = []
        if c.mode == "softcap" and c.softcap_backend != "native":
            selections.append(("tanh_fwd", int(c.softcap_degree), c.softcap_coeff_source))
        if c.mode == "sigmoid_attention" and c.sigmoid_variant == "poly":
            selections.append(("flash_sigmoid_exp2" if bias_aware_d2 else "sigmoid_fwd", degree, c.sigmoid_coeff_source))
            if c.sigmoid_backward_mode == "direct":
                selections.append(("sigmoid_bwd", degree_bwd, c.sigmoid_coeff_source))
            elif degree_bwd != degree:
                family = "flash_sigmoid_exp2" if bias_aware_d2 and degree_bwd == 2 else "sigmoid_fwd"
                selections.append((family, degree_bwd, c.sigmoid_coeff_source))
        if selections:
            audited.extend(runtime["audit_polynomial_selection"](tuple(selections)))
        LOGGER.info("FA4 polynomial audit passed: %s", ", ".join(audited))

    if c.mode == "softmax":
        route = "automatic" if c.exp2_emu_freq is None else c.exp2_emu_freq
        if own_runtime and c.exp2_emu_freq is None:
            route = "automatic -> 0 (all SFU)"
        return ResolvedFA4Config(
            mode="softmax", flash_attn_fwd=fwd, flash_attn_bwd=bwd, exp2_emu_backend=c.exp2_emu_backend,
            exp2_emu_freq=c.exp2_emu_freq, exp2_emu_freq_bwd=c.exp2_emu_freq_bwd, sigmoid_qk_norm=False,
            implementation_summary=(f"FA4 softmax exp2 backend={c.exp2_emu_backend}, forward_freq={route}, "
                                    f"backward_freq={c.exp2_emu_freq_bwd}"))

    if c.mode == "softcap":
        if c.softcap_backend == "native":
            return ResolvedFA4Config(mode="softcap", flash_attn_fwd=fwd, flash_attn_bwd=bwd, softcap=float(c.softcap),
                                     sigmoid_qk_norm=False, implementation_summary="FA4 native SFU tanh softcap")
        paths: list[str] = []
        if c.softcap_backend == "device":
            audit = runtime["audit_attention_handwritten_fast_path"]
            paths.append(audit("tanh_fwd", int(c.softcap_degree), c.softcap_coeff_source))
            if c.softcap_backward_mode == "analytical":
                paths.append(audit("tanh_grad_analytical", int(c.softcap_degree), c.softcap_coeff_source))
        else:
            paths.append(f"CuTe tanh D{int(c.softcap_degree)} {c.softcap_coeff_source}")
        score_mod = runtime["create_softcap_scoremod_backend"](
            c.softcap, degree=c.softcap_degree, backend=c.softcap_backend, coeff_source=c.softcap_coeff_source)
        score_mod_bwd = runtime["create_softcap_scoremod_bwd_backend"](
            c.softcap, degree=c.softcap_degree, backend=c.softcap_backend, backward_mode=c.softcap_backward_mode,
            coeff_source=c.softcap_coeff_source)
        return ResolvedFA4Config(mode="softcap", flash_attn_fwd=fwd, flash_attn_bwd=bwd, score_mod=score_mod,
                                 score_mod_bwd=score_mod_bwd, sigmoid_qk_norm=False,
                                 implementation_summary="; ".join(paths))

    fwd_freq, fwd_res = _sigmoid_route(c.sigmoid_sfu_freq, c.sigmoid_sfu_res, "forward")
    paths = []
    if c.sigmoid_variant == "sfu":
        paths.append("FA4 native SFU sigmoid + algebraic sigmoid gradient")
    elif bias_aware_d2:
        paths.append("FA4 bias-aware D2 exp2 polynomial")
    elif c.sigmoid_poly_backend == "device":
        audit = runtime["audit_attention_handwritten_fast_path"]
        paths.append(audit("flash_sigmoid_direct" if direct else "sigmoid_fwd", degree, c.sigmoid_coeff_source))
        if c.sigmoid_backward_mode == "direct":
            family = "flash_sigmoid_direct_with_grad" if direct and degree_bwd == 4 else "sigmoid_grad"
            paths.append(audit(family, degree_bwd, c.sigmoid_coeff_source))
    return ResolvedFA4Config(
        mode="sigmoid_attention", flash_attn_fwd=fwd, flash_attn_bwd=bwd, sigmoid_attention=True,
        sigmoid_sfu_freq=fwd_freq, sigmoid_sfu_res=fwd_res, sigmoid_sfu_freq_bwd=c.sigmoid_sfu_freq_bwd,
        sigmoid_sfu_res_bwd=c.sigmoid_sfu_res_bwd, sigmoid_use_direct_bwd_poly=(c.sigmoid_backward_mode == "direct"),
        sigmoid_bias=c.sigmoid_bias, sigmoid_poly_backend=c.sigmoid_poly_backend, sigmoid_degree=degree,
        sigmoid_degree_bwd=(degree_bwd if c.sigmoid_degree_bwd is not None else None),
        sigmoid_coeff_source=c.sigmoid_coeff_source, sigmoid_qk_norm=c.sigmoid_qk_norm,
        implementation_summary="; ".join(paths))


def b2_component_configs() -> dict[str, FA4Config]:
    """The native and the polynomial soft-cap configuration of the B2 component probe."""
    return {"native": FA4Config(mode="softcap", softcap=30.0, softcap_backend="native", softcap_backward_mode="native"),
            "polynomial": FA4Config(mode="softcap", softcap=30.0, softcap_backend="device", softcap_degree=4,
                                    softcap_coeff_source="current", softcap_backward_mode="analytical")}


def b3_component_configs(*, sequence_length: int = FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH) -> dict[str, FA4Config]:
    """The SFU and the direct D3/D4 sigmoid configuration of B3; the fitted pair exists for length 4096 only."""
    if int(sequence_length) != FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH:
        raise ValueError(f"B3 direct D3/D4 requires sequence length {FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH}, "
                         f"got {sequence_length}")
    configs = {"native": FA4Config(mode="sigmoid_attention", sigmoid_variant="sfu", sigmoid_sfu_freq=16, sigmoid_sfu_res=16,
                                   sigmoid_qk_norm=True),
               "polynomial": FA4Config(mode="sigmoid_attention", sigmoid_variant="poly", sigmoid_poly_backend="device",
                                       sigmoid_degree=3, sigmoid_degree_bwd=4, sigmoid_coeff_source="current",
                                       sigmoid_backward_mode="direct", sigmoid_sfu_freq=16, sigmoid_sfu_res=0,
                                       sigmoid_qk_norm=True)}
    for config in configs.values():
        validate_fa4_config(config, sequence_length=sequence_length)
    return configs


def softmax_exp2_config(variant: Exp2Variant) -> FA4Config:
    return validate_fa4_config(FA4Config(mode="softmax", exp2_emu_backend=variant.backend,
                                         exp2_emu_freq=variant.forward_frequency,
                                         exp2_emu_freq_bwd=variant.backward_frequency))


def b5_component_configs() -> dict[str, FA4Config]:
    """The three retained routed-exp2 configurations: all-SFU, and two software routes at 1/3 forward, 1/8 backward."""
    variants = (Exp2Variant("native", "d3", 0, 0), Exp2Variant("pwl2_safe_f16", "pwl2_safe_f16", 12, 32),
                Exp2Variant("d2_safe", "d2_safe", 12, 32))
    return {v.name: softmax_exp2_config(v) for v in variants}


_FORWARD_KEYS = ("softcap", "sigmoid_attention", "sigmoid_sfu_freq", "sigmoid_sfu_res", "sigmoid_sfu_freq_bwd",
                 "sigmoid_sfu_res_bwd", "sigmoid_use_direct_bwd_poly", "sigmoid_bias", "sigmoid_poly_backend",
                 "sigmoid_degree", "sigmoid_degree_bwd", "sigmoid_coeff_source", "exp2_emu_backend", "exp2_emu_freq",
                 "exp2_emu_freq_bwd", "score_mod", "score_mod_bwd", "flash_attn_fwd", "flash_attn_bwd")


class _FA4Function(torch.autograd.Function):
    """Forward / backward through the bound runtime; argument order follows the reference's function."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, *settings):
        s = dict(zip(_FORWARD_KEYS, settings))
        for key, fallback in (("sigmoid_sfu_freq_bwd", "sigmoid_sfu_freq"), ("sigmoid_sfu_res_bwd", "sigmoid_sfu_res"),
                              ("sigmoid_degree_bwd", "sigmoid_degree")):
            if s[key] is None:
                s[key] = s[fallback]
        effective_softcap = s["softcap"] if s["score_mod"] is None else 0.0
        out, lse = s["flash_attn_fwd"](
            q, k, v, softmax_scale=softmax_scale, causal=causal, softcap=effective_softcap, score_mod=s["score_mod"],
            sigmoid_attention=s["sigmoid_attention"], sigmoid_sfu_freq=s["sigmoid_sfu_freq"],
            sigmoid_sfu_res=s["sigmoid_sfu_res"], sigmoid_bias=s["sigmoid_bias"],
            sigmoid_poly_backend=s["sigmoid_poly_backend"], sigmoid_degree=s["sigmoid_degree"],
            sigmoid_coeff_source=s["sigmoid_coeff_source"], exp2_emu_backend=s["exp2_emu_backend"],
            exp2_emu_freq=s["exp2_emu_freq"])
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale, ctx.causal, ctx.softcap, ctx.settings = softmax_scale, causal, effective_softcap, s
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        s = ctx.settings
        direct = s["sigmoid_use_direct_bwd_poly"]
        dq, dk, dv = s["flash_attn_bwd"](
            q, k, v, out, dout.contiguous(), lse, ctx.softmax_scale, ctx.causal, ctx.softcap, score_mod=s["score_mod"],
            score_mod_bwd=s["score_mod_bwd"], sigmoid_attention=s["sigmoid_attention"], sigmoid_bias=s["sigmoid_bias"],
            sigmoid_sfu_freq=s["sigmoid_sfu_freq_bwd"], sigmoid_sfu_res=s["sigmoid_sfu_res_bwd"],
            sigmoid_use_direct_bwd_poly=direct, sigmoid_poly_backend=s["sigmoid_poly_backend"],
            sigmoid_degree=(s["sigmoid_degree"] if direct else s["sigmoid_degree_bwd"]),
            sigmoid_gradient_degree=s["sigmoid_degree_bwd"], sigmoid_coeff_source=s["sigmoid_coeff_source"],
            exp2_emu_backend=s["exp2_emu_backend"], exp2_emu_freq=s["exp2_emu_freq_bwd"])
        return (dq, dk, dv, None, None, *([None] * len(_FORWARD_KEYS)))


def _fa4(q, k, v, *, softmax_scale: float | None, causal: bool, config: ResolvedFA4Config) -> torch.Tensor:
    return _FA4Function.apply(q, k, v, softmax_scale, causal, *(getattr(config, key) for key in _FORWARD_KEYS))


class FA4AttentionWrapper(nn.Module):
    """Attention module over (batch, heads, sequence, dim) tensors; always causal, like the reference's wrapper."""

    def __init__(self, config: ResolvedFA4Config, head_dim: int):
        super().__init__()
        self.config = config
        self.head_dim = int(head_dim)
        with_norm = config.sigmoid_attention and config.sigmoid_qk_norm
        self.q_norm: nn.Module | None = nn.RMSNorm(self.head_dim) if with_norm else None
        self.k_norm: nn.Module | None = nn.RMSNorm(self.head_dim) if with_norm else None

    def forward(self, q, k, v, *, score_mod: Callable[..., Any] | None = None, scale: float | None = None, **kwargs: Any):
        if score_mod is not None:
            raise NotImplementedError("external score_mod is unsupported; select it in FA4Config")
        kwargs.pop("enable_gqa", None)
        if kwargs:
            raise TypeError("unsupported FA4 attention kwargs: " + ", ".join(sorted(kwargs)))
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else q.dtype
        to_kernel = lambda t: t.transpose(1, 2).contiguous().to(dtype)
        out = _fa4(to_kernel(q), to_kernel(k), to_kernel(v), softmax_scale=scale, causal=True, config=self.config)
        return out.transpose(1, 2).contiguous()


def build_fa4_module(config: FA4Config, *, head_dim: int, sequence_length: int | None = None) -> FA4AttentionWrapper:
    return FA4AttentionWrapper(resolve_fa4_config(config, sequence_length=sequence_length), head_dim=head_dim)


def patch_attention_modules(model: nn.Module, config: ResolvedFA4Config) -> int:
    """Put a wrapper into every module that has both `inner_attention` and `head_dim`; returns how many."""
    patched = 0
    for module in model.modules():
        if not (hasattr(module, "inner_attention") and hasattr(module, "head_dim")):
            continue
        if isinstance(module.inner_attention, FA4AttentionWrapper):
            continue
        wrapper = FA4AttentionWrapper(config=config, head_dim=module.head_dim)
        parameter = next(module.parameters(), None)
        if parameter is not None:
            wrapper = (wrapper.to(dtype=parameter.dtype) if parameter.device.type == "meta"
                       else wrapper.to(device=parameter.device, dtype=parameter.dtype))
        module.inner_attention = wrapper
        if hasattr(module, "use_flex_attn"):
            module.use_flex_attn = False
        if hasattr(module, "attn_score_modifier"):
            module.attn_score_modifier = None
        patched += 1
    return patched


__all__ = ["DEFAULT_EXP2_VARIANTS", "Exp2Variant", "FA4AttentionWrapper", "FA4Config",
           "FLASH_SIGMOID_DIRECT_SEQUENCE_LENGTH", "ResolvedFA4Config", "SUPPORTED_EXP2_BACKENDS", "SoftcapScoreMod",
           "b200_runtime", "b2_component_configs", "b3_component_configs", "b5_component_configs", "build_fa4_module",
           "parse_exp2_frequency", "parse_exp2_variants", "patch_attention_modules", "resolve_fa4_config",
           "softmax_exp2_config", "validate_fa4_config"]
