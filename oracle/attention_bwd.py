"""CPU restatement of the attention backward for the three modes (test infrastructure, float64 accumulation).

Contract (reference: src/sfu_repro/fa4.py:828-859): `flash_attn_bwd(q, k, v, out, dout, lse, softmax_scale, causal,
softcap, score_mod=..., sigmoid_attention=...) -> (dq, dk, dv)`.  The reference's kernels for it live in a submodule
that is absent, so tiling and rounding points are this build's own; parity against this file is therefore a check of
the mathematics with the same polynomial score-mods, not a pin to reference outputs:

    s = q k^T * scale
    mode 2   P = softmax(s);                       dS = P (dP - delta)
    mode 0   P = softmax(cap * tanhD4(bf16(s/cap))); dS = P (dP - delta) * g(x),  g = d tanhD4/dx (analytical) or 1 - t^2
    mode 1   P = B3(bf16(s)) (no normalisation);   dS = dP * P'(x), P' the coupled derivative of the direct cubic
    mode 3   native twin of mode 0: P = softmax(cap * tanh(s/cap)) with the exact tanh; dS = P (dP - delta) (1 - t^2)
    mode 4   native twin of mode 1: P = sigmoid(s - log n) exactly (no normalisation); dS = dP * P (1 - P)
    dP = dO V^T,  delta = rowsum(dO * O),  dV = bf16(P)^T dO,  dQ = scale * bf16(dS) K,  dK = scale * bf16(dS)^T Q

with P and dS rounded to bf16 where the tensor cores consume them.
"""
from __future__ import annotations

import numpy as np

from . import oracle


def _bf16_round(x: np.ndarray) -> np.ndarray:
    return oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x.astype(np.float32))).astype(np.float64)


def _tanh_program():
    idx = oracle.find_program("TANH_FWD_D4", oracle.BF16)
    row = oracle.program_table()[idx]
    coeffs = oracle.bf16_bits_to_f32(np.array(row["coeffs"][:4], dtype=np.uint16)).astype(np.float64)
    clamp = float(oracle.bf16_bits_to_f32(np.array([row["clamp"]], dtype=np.uint16))[0])
    return idx, coeffs, clamp


def attention_fwd_bwd(q_bits, k_bits, v_bits, dout_bits, mode: int, causal: bool, scale: float, softcap: float = 0.0,
                      log2_n: int = 12, softcap_grad: int = 0):
    """bf16 bit patterns [B,S,H,D] in; float64 (out, lse, dq, dk, dv) out."""
    q = oracle.bf16_bits_to_f32(q_bits).astype(np.float64)
    k = oracle.bf16_bits_to_f32(k_bits).astype(np.float64)
    v = oracle.bf16_bits_to_f32(v_bits).astype(np.float64)
    do = oracle.bf16_bits_to_f32(dout_bits).astype(np.float64)
    B, S, Hq, D = q.shape
    Hk = k.shape[2]
    group = Hq // Hk
    out = np.zeros_like(q)
    lse = np.zeros((B, Hq, S))
    dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    mask = np.tril(np.ones((S, S), dtype=bool)) if causal else np.ones((S, S), dtype=bool)
    tanh_idx, tanh_c, tanh_clamp = _tanh_program()
    for b in range(B):
        for h in range(Hq):
            hk = h // group
            raw = q[b, :, h, :] @ k[b, :, hk, :].T
            g = None
            if mode == 1:
                x_bits = oracle.f32_to_bf16_bits((raw * scale).astype(np.float32))
                p_bits, grad_bits = oracle.b3_direct(x_bits.ravel(), log2_n, with_grad=True)
                p = oracle.bf16_bits_to_f32(p_bits).astype(np.float64).reshape(S, S) * mask
                grad = oracle.bf16_bits_to_f32(grad_bits).astype(np.float64).reshape(S, S) * mask
                p_mma = p                                    # already bf16 values
            elif mode == 4:
                p = 1.0 / (1.0 + np.exp(log2_n * np.log(2.0) - raw * scale)) * mask
                grad = p * (1.0 - p)
                p_mma = _bf16_round(p)
            else:
                if mode == 3:
                    t = np.tanh(raw * (scale / softcap))
                    s = softcap * t
                    g = 1.0 - t * t
                elif mode == 0:
                    x_bits = oracle.f32_to_bf16_bits((raw * (scale / softcap)).astype(np.float32))
                    t_bits = oracle.unary(tanh_idx, x_bits.ravel())
                    t = oracle.bf16_bits_to_f32(t_bits).astype(np.float64).reshape(S, S)
                    s = softcap * t
                    if softcap_grad == 1:
                        g = 1.0 - t * t
                    else:
                        ax = np.abs(oracle.bf16_bits_to_f32(x_bits).astype(np.float64))
                        c = np.minimum(ax, tanh_clamp)
                        g = tanh_c[0] + c * (2 * tanh_c[1] + c * (3 * tanh_c[2] + c * 4 * tanh_c[3]))
                        g = np.where((ax < tanh_clamp) & (np.abs(t) < 1.0), g, 0.0)
                else:
                    s = raw * scale
                s = np.where(mask, s, -np.inf)
                m = s.max(axis=1, keepdims=True)
                e = np.exp(s - m)
                lse[b, h] = (m + np.log(e.sum(axis=1, keepdims=True)))[:, 0]
                p = e / e.sum(axis=1, keepdims=True)
                p_mma = _bf16_round(p)
            o = p_mma @ v[b, :, hk, :]
            out[b, :, h, :] = o
            dp = do[b, :, h, :] @ v[b, :, hk, :].T
            if mode in (1, 4):
                ds = dp * grad
            else:
                delta = (do[b, :, h, :] * _bf16_round(o)).sum(axis=1, keepdims=True)
                ds = p * (dp - delta)
                if g is not None:
                    ds = ds * g
            ds_mma = _bf16_round(ds)
            dv[b, :, hk, :] += p_mma.T @ do[b, :, h, :]
            dq[b, :, h, :] = scale * (ds_mma @ k[b, :, hk, :])
            dk[b, :, hk, :] += scale * (ds_mma.T @ q[b, :, h, :])
    return out, lse, dq, dk, dv
