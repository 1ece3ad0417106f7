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

// The same function with fewer half-rate ALU operations, for the attention warps: both cubics are evaluated on
// the FMA pipe and ONE select picks the lane's row afterwards (identical arithmetic per lane, so identical bits),
// and the lower clamp is dropped: below -6 the low-row cubic stays negative all the way to -inf (its derivative is
// positive there), so the final max(., +0) returns the same +0 the clamped evaluation returns.
__device__ __forceinline__ uint32_t b3_direct_select_late(uint32_t x, const B3Words& k) {
    using P = Pk<kBf16>;
    const uint32_t mask = P::ge_mask(x, k.split);
    const uint32_t c = P::min(x, k.clamp_hi);
    uint32_t lo = P::fma(c, k.lo[3], k.lo[2]);
    uint32_t hi = P::fma(c, k.hi[3], k.hi[2]);
    lo = P::fma(c, lo, k.lo[1]);
    hi = P::fma(c, hi, k.hi[1]);
    // The floor at +0 rides on the last multiply-add of each row (max(select(hi, lo), 0) = select(max(hi, 0), max(lo, 0));
    // neither row can end in -0, its last addend being a non-zero constant), which saves the separate maximum.
    lo = P::fma_relu(c, lo, k.lo[0]);
    hi = P::fma_relu(c, hi, k.hi[0]);
    return select_bits(mask, hi, lo);
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

// The pair (value, coupled derivative) with the late select of b3_direct_select_late: both rows' cubics and both rows'
// derivative factors on the FMA pipe, one select each, no lower clamp.  Below -6 the value is +0 and the low-row factor
// 1 - slope |x| stays positive and finite for every finite x, so the product is the same +0 the clamped form gives.  The
// one input that differs is -inf: its factor is +inf and 0 * inf is NaN where the clamped form returns +0.  Callers that
// can meet an infinite score (an overflowed dot product) therefore convert their fp32 scores with
// Sfu<kBf16>::pack_satfinite, which costs nothing and maps -inf to the largest finite negative value (result +0, +0).
// For the attention backward, whose score-mod warps are bound by the half-rate ALU pipe.
__device__ __forceinline__ uint32_t b3_direct_with_grad_select_late(uint32_t x, const B3Words& k, uint32_t& grad) {
    using P = Pk<kBf16>;
    const uint32_t mask = P::ge_mask(x, k.split);
    const uint32_t c = P::min(x, k.clamp_hi);
    uint32_t lo = P::fma(c, k.lo[3], k.lo[2]);
    uint32_t hi = P::fma(c, k.hi[3], k.hi[2]);
    lo = P::fma(c, lo, k.lo[1]);
    hi = P::fma(c, hi, k.hi[1]);
    lo = P::fma_relu(c, lo, k.lo[0]);
    hi = P::fma_relu(c, hi, k.hi[0]);
    const uint32_t v = select_bits(mask, hi, lo);
    const uint32_t factor = select_bits(mask, P::fma(c, k.grad_hi[1], k.grad_hi[0]), P::fma(c, k.grad_lo[1], k.grad_lo[0]));
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

// ---------------------------------------------------------------------------------------------------------------
// Full-range 2^a in fp32 on the FMA pipe: the software exponentials that take a share of the soft-max work off the
// special-function unit (reference: autonumerics_zero/cuda_benchmarks/benchmark_exp2_pwl2.cu:106-198, FullDegree3 and
// FullPwl2Hinge; the same sequences, operation for operation, so that results agree bit for bit):
//   a'  = max(a, -127)
//   xr  = a' + 1.5 * 2^23  rounded TOWARDS MINUS INFINITY (the low mantissa bits of xr now hold n = floor(a'))
//   f   = a' - (xr - 1.5 * 2^23)             in [0, 1), exact
//   D3:   p = 1 + f (c1 + f (c2 + f c3))                         cubic, relative error 8.8e-5
//   PWL2: p = k0 + k1 f + k2 max(f - 1/2, 0)                     continuous two-piece line, relative error 2.1e-2
//   2^a = bits(p) + (bits(xr) << 23)         (the shift drops the magic constant's own bits, n lands on the exponent)
// Every step is one IEEE operation (flush-to-zero as in the reference; no step here meets a subnormal for a <= 127).
// Two more fractional evaluators keep the same reduction and reconstruction and preserve both endpoints (p(0) = 1,
// p(1) = 2), which an online soft-max needs for its rescaling steps to compose (reference:
// extras/paper/manuscript/appendix_exp2.tex:18-33 fits, :74-80 packed fp16 constants; the reference's own instruction
// listing for them sits in its attention submodule, so the operation order below is this library's):
//   D2_SAFE:       p = 1 + a f + (1 - a) f^2, a = 0.6602339719      two fp32 multiply-adds, relative error 2.7e-3
//   PWL2_SAFE_F16: p = 1 + A f + C max(f - 1/2, 0) on a packed fp16 pair, A = 0.7978515625, C = 0.40380859375:
//                  f -> fp16, subtract, maximum, two fp16 multiply-adds, back to fp32; relative error 1.1e-2
enum Exp2Full : int { kExp2FullD3 = 0, kExp2FullPwl2 = 1, kExp2FullD2Safe = 2, kExp2FullPwl2SafeF16 = 3 };
constexpr float kExp2Magic = 12582912.0f;            // 0x4B400000
// Lowest argument: -127 for the cubic (p >= 1, so the sum of bit patterns ends exactly at +0); -126 for the two-piece
// line, which starts at p = 0.989 < 1: one exponent lower its bit pattern would wrap to a negative NaN pattern (the
// reference clamps both at -127 and only feeds the line arguments above that; masked soft-max scores are -inf).
template <int KIND> constexpr float kExp2Floor = KIND == 1 ? -126.0f : -127.0f;
constexpr float kExp2D3C1 = 0.6951461434364319f;     // 0x3F31F519
constexpr float kExp2D3C2 = 0.22756439447402954f;    // 0x3E6906A4
constexpr float kExp2D3C3 = 0.07711908966302872f;    // 0x3D9DF09D
constexpr float kExp2PwlK0 = 0.9894611835479736f;    // 0x3F7D4D54
constexpr float kExp2PwlK1 = 0.820852518081665f;     // 0x3F522364
constexpr float kExp2PwlK2 = 0.34246066212654114f;   // 0x3EAF5701
constexpr float kExp2D2A = 0.6602339719f;            // endpoint-preserving quadratic: a
constexpr float kExp2D2B = 0.3397660281f;            //                                1 - a

// 2^f for a pair f0, f1 in [0, 1) on packed fp16 lanes (endpoint-preserving two-piece line), widened to fp32
__device__ __forceinline__ void exp2_fraction_pwl2_f16(float f0, float f1, float& p0, float& p1) {
    const uint32_t fh = Sfu<kFp16>::pack(f0, f1);
    const uint32_t ph = exp2_hinge(fh, Exp2Words{0x3a623a62u, 0x3c003c00u, 0x36763676u});   // A, 1, C in fp16
    p0 = Sfu<kFp16>::lo(ph);
    p1 = Sfu<kFp16>::hi(ph);
}

template <int KIND>
__device__ __forceinline__ float exp2_full(float a) {
    a = fmaxf(a, kExp2Floor<KIND>);
    const float xr = __fadd_rd(a, kExp2Magic);
    const float f = __fsub_rn(a, __fsub_rn(xr, kExp2Magic));
    float p;
    if constexpr (KIND == kExp2FullD3) {
        p = __fmaf_rn(f, kExp2D3C3, kExp2D3C2);
        p = __fmaf_rn(p, f, kExp2D3C1);
        p = __fmaf_rn(p, f, 1.0f);
    } else if constexpr (KIND == kExp2FullPwl2) {
        const float h = fmaxf(__fsub_rn(f, 0.5f), 0.0f);
        p = __fmaf_rn(f, kExp2PwlK1, kExp2PwlK0);
        p = __fmaf_rn(h, kExp2PwlK2, p);
    } else if constexpr (KIND == kExp2FullD2Safe) {
        p = __fmaf_rn(f, kExp2D2B, kExp2D2A);
        p = __fmaf_rn(p, f, 1.0f);
    } else {
        float unused;
        exp2_fraction_pwl2_f16(f, f, p, unused);
    }
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(xr) << 23));
}

// The same on two values at once with the packed fp32 instructions (two lanes per issue slot).
template <int KIND>
__device__ __forceinline__ void exp2_full_x2(float a0, float a1, float& e0, float& e1) {
    a0 = fmaxf(a0, kExp2Floor<KIND>);
    a1 = fmaxf(a1, kExp2Floor<KIND>);
    uint32_t p0, p1, x0, x1;
    if constexpr (KIND == kExp2FullD3) {
        asm("{\n\t.reg .b64 a, m, xr, n, f, p, c;\n\t"
            "mov.b64 a, {%4, %5};\n\t"
            "mov.b64 m, {%6, %6};\n\t"
            "add.rm.ftz.f32x2 xr, a, m;\n\t"
            "sub.rn.ftz.f32x2 n, xr, m;\n\t"
            "sub.rn.ftz.f32x2 f, a, n;\n\t"
            "mov.b64 p, {%7, %7};\n\t"
            "mov.b64 c, {%8, %8};\n\t"
            "fma.rn.ftz.f32x2 p, f, p, c;\n\t"
            "mov.b64 c, {%9, %9};\n\t"
            "fma.rn.ftz.f32x2 p, p, f, c;\n\t"
            "mov.b64 c, {%10, %10};\n\t"
            "fma.rn.ftz.f32x2 p, p, f, c;\n\t"
            "mov.b64 {%0, %1}, p;\n\t"
            "mov.b64 {%2, %3}, xr;\n\t}"
            : "=r"(p0), "=r"(p1), "=r"(x0), "=r"(x1)
            : "f"(a0), "f"(a1), "f"(kExp2Magic), "f"(kExp2D3C3), "f"(kExp2D3C2), "f"(kExp2D3C1), "f"(1.0f));
    } else if constexpr (KIND == kExp2FullD2Safe) {
        asm("{\n\t.reg .b64 a, m, xr, n, f, p, c;\n\t"
            "mov.b64 a, {%4, %5};\n\t"
            "mov.b64 m, {%6, %6};\n\t"
            "add.rm.ftz.f32x2 xr, a, m;\n\t"
            "sub.rn.ftz.f32x2 n, xr, m;\n\t"
            "sub.rn.ftz.f32x2 f, a, n;\n\t"
            "mov.b64 p, {%7, %7};\n\t"
            "mov.b64 c, {%8, %8};\n\t"
            "fma.rn.ftz.f32x2 p, f, p, c;\n\t"
            "mov.b64 c, {%9, %9};\n\t"
            "fma.rn.ftz.f32x2 p, p, f, c;\n\t"
            "mov.b64 {%0, %1}, p;\n\t"
            "mov.b64 {%2, %3}, xr;\n\t}"
            : "=r"(p0), "=r"(p1), "=r"(x0), "=r"(x1)
            : "f"(a0), "f"(a1), "f"(kExp2Magic), "f"(kExp2D2B), "f"(kExp2D2A), "f"(1.0f));
    } else if constexpr (KIND == kExp2FullPwl2SafeF16) {
        float f0, f1, q0, q1;
        asm("{\n\t.reg .b64 a, m, xr, n, f;\n\t"
            "mov.b64 a, {%4, %5};\n\t"
            "mov.b64 m, {%6, %6};\n\t"
            "add.rm.ftz.f32x2 xr, a, m;\n\t"
            "sub.rn.ftz.f32x2 n, xr, m;\n\t"
            "sub.rn.ftz.f32x2 f, a, n;\n\t"
            "mov.b64 {%0, %1}, f;\n\t"
            "mov.b64 {%2, %3}, xr;\n\t}"
            : "=f"(f0), "=f"(f1), "=r"(x0), "=r"(x1) : "f"(a0), "f"(a1), "f"(kExp2Magic));
        exp2_fraction_pwl2_f16(f0, f1, q0, q1);
        p0 = __float_as_uint(q0);
        p1 = __float_as_uint(q1);
    } else {
        float f0, f1;
        asm("{\n\t.reg .b64 a, m, xr, n, f;\n\t"
            "mov.b64 a, {%4, %5};\n\t"
            "mov.b64 m, {%6, %6};\n\t"
            "add.rm.ftz.f32x2 xr, a, m;\n\t"
            "sub.rn.ftz.f32x2 n, xr, m;\n\t"
            "sub.rn.ftz.f32x2 f, a, n;\n\t"
            "mov.b64 {%0, %1}, f;\n\t"
            "mov.b64 {%2, %3}, xr;\n\t}"
            : "=f"(f0), "=f"(f1), "=r"(x0), "=r"(x1) : "f"(a0), "f"(a1), "f"(kExp2Magic));
        const float h0 = fmaxf(__fsub_rn(f0, 0.5f), 0.0f), h1 = fmaxf(__fsub_rn(f1, 0.5f), 0.0f);
        asm("{\n\t.reg .b64 f, h, p, c;\n\t"
            "mov.b64 f, {%2, %3};\n\t"
            "mov.b64 h, {%4, %5};\n\t"
            "mov.b64 p, {%6, %6};\n\t"
            "mov.b64 c, {%7, %7};\n\t"
            "fma.rn.ftz.f32x2 p, f, p, c;\n\t"
            "mov.b64 c, {%8, %8};\n\t"
            "fma.rn.ftz.f32x2 p, h, c, p;\n\t"
            "mov.b64 {%0, %1}, p;\n\t}"
            : "=r"(p0), "=r"(p1) : "f"(f0), "f"(f1), "f"(h0), "f"(h1), "f"(kExp2PwlK1), "f"(kExp2PwlK0), "f"(kExp2PwlK2));
    }
    e0 = __uint_as_float(p0 + (x0 << 23));
    e1 = __uint_as_float(p1 + (x1 << 23));
}

// ---- two fp32 lanes per instruction (add / sub / mul / fma .f32x2): one issue slot for a pair of keys ------------
// (o0, o1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void mul2(float a0, float a1, float b0, float b1, float& o0, float& o1) {
    asm("{\n\t.reg .b64 a, b, r;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\t"
        "mul.rn.f32x2 r, a, b;\n\tmov.b64 {%0, %1}, r;\n\t}"
        : "=f"(o0), "=f"(o1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// (o0, o1) = (a0, a1) - (b0, b1)
__device__ __forceinline__ void sub2(float a0, float a1, float b0, float b1, float& o0, float& o1) {
    asm("{\n\t.reg .b64 a, b, r;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\t"
        "sub.rn.f32x2 r, a, b;\n\tmov.b64 {%0, %1}, r;\n\t}"
        : "=f"(o0), "=f"(o1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// (o0, o1) = (a0, a1) * (b0, b1) + (c0, c1)
__device__ __forceinline__ void fma2(float a0, float a1, float b0, float b1, float c0, float c1, float& o0, float& o1) {
    asm("{\n\t.reg .b64 a, b, c, r;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmov.b64 c, {%6, %7};\n\t"
        "fma.rn.f32x2 r, a, b, c;\n\tmov.b64 {%0, %1}, r;\n\t}"
        : "=f"(o0), "=f"(o1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
// the two bf16 lanes of a word as fp32 (a shift and a mask)
__device__ __forceinline__ void unpack_bf16x2(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}

}  // namespace fpt
