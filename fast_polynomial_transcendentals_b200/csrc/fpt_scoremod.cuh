// Score-mod evaluators shared by the isolated element-wise kernels and the attention kernel.
#pragma once

#include "fpt_packed.cuh"

namespace fpt {

// ---- B3: direct piecewise-cubic sigmoid on the raw score ----------------------------------------
// p(x) ~ sigmoid(x - log n).  x is compared with the split on the UNCLAMPED bf16 score (ordered: NaN selects
// the low row), clamped to [-6, 6], a cubic with row-selected coefficients is evaluated by three packed
// FMAs from the highest coefficient down, and the result is floored at +0.  The deployed coefficients are
// fitted for n = 4096 and pre-scaled by 2^-12; another power-of-two length shifts them exactly.
struct B3Words {
    uint32_t split, clamp_hi, clamp_lo;
    uint32_t lo[4], hi[4];       // c0..c3 for x < split / x >= split
    uint32_t grad_lo[2], grad_hi[2];  // derivative factor: intercept, slope
};

inline B3Words b3_words(int log2_n) {
    static const uint16_t row0[4] = {0x3980, 0x3987, 0x3909, 0x37e8};
    static const uint16_t row1[4] = {0xbb09, 0x3b8c, 0xbb11, 0x3a09};
    B3Words k;
    k.split = 0x3fa03fa0u;
    k.clamp_hi = 0x40c040c0u;
    k.clamp_lo = 0xc0c0c0c0u;
    const int down = log2_n - 12;
    for (int i = 0; i < 4; ++i) {
        k.lo[i] = uint32_t(uint16_t(row0[i] - (down << 7))) * 0x00010001u;
        k.hi[i] = uint32_t(uint16_t(row1[i] - (down << 7))) * 0x00010001u;
    }
    k.grad_lo[0] = 0x3f803f80u; k.grad_lo[1] = 0xbc10bc10u;
    k.grad_hi[0] = 0x3f813f81u; k.grad_hi[1] = 0xbb38bb38u;
    return k;
}

__device__ __forceinline__ uint32_t select_bits(uint32_t mask, uint32_t when_set, uint32_t when_clear) {
    return (mask & when_set) | (~mask & when_clear);
}

__device__ __forceinline__ uint32_t b3_direct_core(uint32_t x, const B3Words& k, uint32_t& mask, uint32_t& c) {
    using P = Pk<kBf16>;
    mask = P::ge_mask(x, k.split);
    c = P::max(P::min(x, k.clamp_hi), k.clamp_lo);
    uint32_t v = select_bits(mask, k.hi[3], k.lo[3]);
    v = P::fma(c, v, select_bits(mask, k.hi[2], k.lo[2]));
    v = P::fma(c, v, select_bits(mask, k.hi[1], k.lo[1]));
    v = P::fma(c, v, select_bits(mask, k.hi[0], k.lo[0]));
    return P::max(v, 0u);
}

__device__ __forceinline__ uint32_t b3_direct(uint32_t x, const B3Words& k) {
    uint32_t mask, c;
    return b3_direct_core(x, k, mask, c);
}

// value and value * (intercept + slope * clamp(x)), the coupled derivative of the deployed pair
__device__ __forceinline__ uint32_t b3_direct_with_grad(uint32_t x, const B3Words& k, uint32_t& grad) {
    using P = Pk<kBf16>;
    uint32_t mask, c;
    const uint32_t v = b3_direct_core(x, k, mask, c);
    const uint32_t factor = P::fma(c, select_bits(mask, k.grad_hi[1], k.grad_lo[1]),
                                   select_bits(mask, k.grad_hi[0], k.grad_lo[0]));
    grad = P::mul(v, factor);
    return v;
}

// ---- fractional exp2, x in [0, 1): two-segment hinge  p(x) = offset + slope*x + delta*max(x - 1/2, 0) --
struct Exp2Words {
    uint32_t slope, offset, delta;
};

inline Exp2Words exp2_words(bool endpoint_preserving) {
    // least-squares constants of the reference benchmark / endpoint-preserving constants (p(0)=1, p(1)=2)
    return endpoint_preserving ? Exp2Words{0x3a623a62u, 0x3c003c00u, 0x36763676u}
                               : Exp2Words{0x3a913a91u, 0x3bea3beau, 0x357b357bu};
}

__device__ __forceinline__ uint32_t exp2_hinge(uint32_t x, const Exp2Words& k) {
    using P = Pk<kFp16>;
    const uint32_t hinge = P::max(P::sub(x, 0x38003800u), 0u);
    const uint32_t base = P::fma(x, k.slope, k.offset);
    return P::fma(hinge, k.delta, base);
}

}  // namespace fpt
