"""Shared helpers for the tests: seeded inputs, bit views, reference-library calls."""
from __future__ import annotations

import ctypes

import numpy as np

SPECIALS_BF16 = [0x0000, 0x8000, 0x7F80, 0xFF80, 0x7FC0, 0x0001, 0x007F, 0x8001, 0x807F]
SPECIALS_FP16 = [0x0000, 0x8000, 0x7C00, 0xFC00, 0x7E00, 0x0001, 0x03FF, 0x8001, 0x83FF]


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def uniform_bits(n: int, lo: float, hi: float, dtype: str, seed: int = 1234, special_fraction: float = 0.01):
    """U[lo,hi) in fp32 rounded to the 16-bit format, with a fraction of positions overwritten
    cyclically by +-0, +-inf, NaN and subnormals (the configuration-1 recipe)."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(lo, hi, size=n).astype(np.float32)
    bits = f32_to_bf16_bits(x) if dtype == "bf16" else x.astype(np.float16).view(np.uint16)
    if special_fraction > 0 and n > 0:
        k = max(1, int(n * special_fraction))
        pos = rng.permutation(n)[:k]
        sp = np.array(SPECIALS_BF16 if dtype == "bf16" else SPECIALS_FP16, dtype=np.uint16)
        bits[pos] = sp[np.arange(k) % sp.size]
    return bits


def normal_bits(n: int, std: float, dtype: str, seed: int = 1234):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * std).astype(np.float32)
    return f32_to_bf16_bits(x) if dtype == "bf16" else x.astype(np.float16).view(np.uint16)


def to_device(bits: np.ndarray, dtype: str, device):
    import torch
    t = torch.from_numpy(bits.view(np.int16).copy()).to(device)
    return t.view(torch.bfloat16 if dtype == "bf16" else torch.float16)


def to_bits(t) -> np.ndarray:
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def assert_bits_equal(got: np.ndarray, want: np.ndarray, what: str, inputs: np.ndarray | None = None):
    got, want = np.asarray(got).ravel(), np.asarray(want).ravel()
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    bad = np.nonzero(got != want)[0]
    if bad.size:
        show = []
        for i in bad[:8]:
            item = f"[{i}] got 0x{got[i]:04x} want 0x{want[i]:04x}"
            if inputs is not None and inputs.size == got.size:
                item += f" in 0x{np.asarray(inputs).ravel()[i]:04x}"
            show.append(item)
        raise AssertionError(f"{what}: {bad.size} of {got.size} lanes differ: " + "; ".join(show))


def ref_call(lib, symbol: str, *args):
    """Call a `launch_*` symbol of the reference kernel library: pointers as c_void_p, ints as c_int,
    stream last (NULL = legacy default stream)."""
    fn = getattr(lib, symbol)
    fn.restype = None
    conv = []
    for a in args:
        conv.append(ctypes.c_void_p(a.data_ptr()) if hasattr(a, "data_ptr") else ctypes.c_int(int(a)))
    fn(*conv, ctypes.c_void_p(0))
