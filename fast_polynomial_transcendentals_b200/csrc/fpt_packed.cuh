// Packed 16-bit lane arithmetic and the polynomial program shapes, for sm_100a.
//
// Every arithmetic step is an explicit `.rn` PTX instruction on a 32-bit word
// holding two fp16 or two bf16 lanes, so the compiler can neither contract a
// multiply into a following add nor reorder roundings: the result of a kernel
// is defined by the instruction sequence written here and nothing else.
// Coefficients arrive as 32-bit words with the 16-bit pattern duplicated in
// both lanes (kernel parameters, i.e. constant-bank operands of HFMA2).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace fpt {

enum Dtype : int { kFp16 = 0, kBf16 = 1 };

// Program shapes; t = min(|x|, clamp), h = t*(c1 + t*(c2 + ...)), s = sign bit of x.
enum Shape : int {
    kOddHalf = 0,   // 0.5 + s*h              sigmoid fwd, swish bwd, gelu bwd
    kOdd = 1,       // s*h                    tanh fwd (fp16), erf fwd
    kOddSat = 2,    // s*min(h, 1)            tanh fwd (bf16)
    kSwish = 3,     // fma(|x|, h, 0.5*x)     swish fwd, direct form
    kXmulHalf = 4,  // x*(0.5 + s*h)          gelu fwd, composed swish fwd
    kEven = 5,      // c0 + t*(c1 + t*(...))  sigmoid / tanh bwd
    kAlgSig = 6,    // y*(1 - y)
    kAlgTanh = 7,   // 1 - y*y
    kShapeCount = 8
};

struct ProgramWords {
    uint32_t clamp;
    uint32_t c[7];
};

template <int DT>
struct Pk;

#define FPT_PK_OPS(DT, SUF)                                                                         \
    template <>                                                                                     \
    struct Pk<DT> {                                                                                 \
        static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {        \
            uint32_t d;                                                                             \
            asm("fma.rn." SUF " %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));               \
            return d;                                                                               \
        }                                                                                           \
        /* max(a * b + c, +0) in the multiply-add itself */                                          \
        static __device__ __forceinline__ uint32_t fma_relu(uint32_t a, uint32_t b, uint32_t c) {   \
            uint32_t d;                                                                             \
            asm("fma.rn.relu." SUF " %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));          \
            return d;                                                                               \
        }                                                                                           \
        static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {                    \
            uint32_t d;                                                                             \
            asm("mul.rn." SUF " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                           \
            return d;                                                                               \
        }                                                                                           \
        static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {                    \
            uint32_t d;                                                                             \
            asm("add.rn." SUF " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                           \
            return d;                                                                               \
        }                                                                                           \
        static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {                    \
            uint32_t d;                                                                             \
            asm("sub.rn." SUF " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                           \
            return d;                                                                               \
        }                                                                                           \
        static __device__ __forceinline__ uint32_t min(uint32_t a, uint32_t b) {                    \
            uint32_t d;                                                                             \
            asm("min." SUF " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                              \
            return d;                                                                               \
        }                                                                                           \
        /* min(|a|, b): the absolute value as an instruction of its own, which the assembler can fold into the    */ \
        /* comparison as a source modifier (one ALU-pipe instruction less than masking the sign bits first)     */ \
        static __device__ __forceinline__ uint32_t min_abs(uint32_t a, uint32_t b) {                \
            uint32_t d;                                                                             \
            asm("{\n\t.reg .b32 t;\n\tabs." SUF " t, %1;\n\tmin." SUF " %0, t, %2;\n\t}" : "=r"(d) : "r"(a), "r"(b)); \
            return d;                                                                               \
        }                                                                                           \
        static __device__ __forceinline__ uint32_t max(uint32_t a, uint32_t b) {                    \
            uint32_t d;                                                                             \
            asm("max." SUF " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                              \
            return d;                                                                               \
        }                                                                                           \
        /* per-lane 0xffff where a >= b (ordered: false on NaN) */                                  \
        static __device__ __forceinline__ uint32_t ge_mask(uint32_t a, uint32_t b) {                \
            uint32_t d;                                                                             \
            asm("set.ge.u32." SUF " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                       \
            return d;                                                                               \
        }                                                                                           \
    };

FPT_PK_OPS(kFp16, "f16x2")
FPT_PK_OPS(kBf16, "bf16x2")
#undef FPT_PK_OPS

template <int DT>
struct Consts;
template <>
struct Consts<kFp16> {
    static constexpr uint32_t half = 0x38003800u, one = 0x3c003c00u;
};
template <>
struct Consts<kBf16> {
    static constexpr uint32_t half = 0x3f003f00u, one = 0x3f803f80u;
};

constexpr uint32_t kSignMask = 0x80008000u;

// One polynomial program on two lanes.
template <int DT, int SHAPE, int DEG>
__device__ __forceinline__ uint32_t eval_program(uint32_t x, const ProgramWords& p) {
    using P = Pk<DT>;
    if constexpr (SHAPE == kAlgSig) {
        return P::mul(x, P::sub(Consts<DT>::one, x));
    } else if constexpr (SHAPE == kAlgTanh) {
        return P::sub(Consts<DT>::one, P::mul(x, x));
    } else {
        const uint32_t sign = x & kSignMask;
        const uint32_t a = x & ~kSignMask;
        const uint32_t t = P::min_abs(x, p.clamp);
        if constexpr (SHAPE == kEven) {
            uint32_t r = P::fma(t, p.c[DEG], p.c[DEG - 1]);
#pragma unroll
            for (int k = DEG - 2; k >= 0; --k) r = P::fma(t, r, p.c[k]);
            return r;
        } else {
            uint32_t h = P::fma(t, p.c[DEG - 1], p.c[DEG - 2]);
#pragma unroll
            for (int k = DEG - 3; k >= 0; --k) h = P::fma(t, h, p.c[k]);
            h = P::mul(t, h);
            if constexpr (SHAPE == kOdd) return h ^ sign;
            if constexpr (SHAPE == kOddSat) return P::min(h, Consts<DT>::one) ^ sign;
            if constexpr (SHAPE == kOddHalf) return P::add(Consts<DT>::half, h ^ sign);
            if constexpr (SHAPE == kXmulHalf) return P::mul(x, P::add(Consts<DT>::half, h ^ sign));
            if constexpr (SHAPE == kSwish) return P::fma(a, h, P::mul(Consts<DT>::half, x));
        }
    }
    return 0;
}

// ---- MUFU (special function unit) twins used as native controls ------------------------------

template <int DT>
struct Sfu;
template <>
struct Sfu<kFp16> {
    static __device__ __forceinline__ uint32_t ex2(uint32_t x) {
        uint32_t d;
        asm("ex2.approx.f16x2 %0, %1;" : "=r"(d) : "r"(x));
        return d;
    }
    static __device__ __forceinline__ uint32_t tanh(uint32_t x) {
        uint32_t d;
        asm("tanh.approx.f16x2 %0, %1;" : "=r"(d) : "r"(x));
        return d;
    }
    static __device__ __forceinline__ float lo(uint32_t x) {
        float f;
        asm("{.reg .f16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, l;}" : "=f"(f) : "r"(x));
        return f;
    }
    static __device__ __forceinline__ float hi(uint32_t x) {
        float f;
        asm("{.reg .f16 l, h; mov.b32 {l, h}, %1; cvt.f32.f16 %0, h;}" : "=f"(f) : "r"(x));
        return f;
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t d;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
        return d;
    }
    static constexpr uint32_t log2e = 0x3dc53dc5u;      // 1.4427 in fp16
    static constexpr uint32_t neg_log2e = 0xbdc5bdc5u;
};
template <>
struct Sfu<kBf16> {
    static __device__ __forceinline__ uint32_t ex2(uint32_t x) {
        uint32_t d;
        asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(d) : "r"(x));
        return d;
    }
    static __device__ __forceinline__ uint32_t tanh(uint32_t x) {
        uint32_t d;
        asm("tanh.approx.bf16x2 %0, %1;" : "=r"(d) : "r"(x));
        return d;
    }
    static __device__ __forceinline__ float lo(uint32_t x) { return __uint_as_float(x << 16); }
    static __device__ __forceinline__ float hi(uint32_t x) { return __uint_as_float(x & 0xffff0000u); }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t d;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
        return d;
    }
    // the same conversion with infinities replaced by the largest finite value of their sign (NaN stays NaN)
    static __device__ __forceinline__ uint32_t pack_satfinite(float lo, float hi) {
        uint32_t d;
        asm("cvt.rn.satfinite.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
        return d;
    }
    static constexpr uint32_t log2e = 0x3fb93fb9u;      // 1.4453 in bf16
    static constexpr uint32_t neg_log2e = 0xbfb9bfb9u;
};

__device__ __forceinline__ float mufu_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mufu_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mufu_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Native controls evaluate in fp32 per lane: two MUFU ops (ex2 + rcp) per element for
// sigmoid-like functions, one (tanh) for tanh, and round once to the lane format.
enum NativeFn : int { kNatSigmoid = 0, kNatTanh = 1, kNatSwish = 2, kNatSwishGrad = 3, kNatSigmoidGrad = 4,
                      kNatTanhGrad = 5, kNatGelu = 6, kNatGeluGrad = 7, kNatErf = 8 };

template <int FN>
__device__ __forceinline__ float native_scalar(float x) {
    if constexpr (FN == kNatTanh) return mufu_tanh(x);
    if constexpr (FN == kNatTanhGrad) { float y = mufu_tanh(x); return fmaf(-y, y, 1.0f); }
    if constexpr (FN == kNatGelu || FN == kNatGeluGrad || FN == kNatErf) {
        // tanh form of erf-based quantities is NOT used: erff keeps the control exact enough to
        // serve as an accuracy yardstick as well as a timing one.
        if constexpr (FN == kNatErf) return erff(x);
        const float phi = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
        if constexpr (FN == kNatGelu) return x * phi;
        return phi + x * 0.3989422804014327f * mufu_ex2(-0.72134752044448170368f * x * x);
    }
    const float sig = mufu_rcp(1.0f + mufu_ex2(-1.4426950408889634f * x));
    if constexpr (FN == kNatSigmoid) return sig;
    if constexpr (FN == kNatSwish) return x * sig;
    if constexpr (FN == kNatSigmoidGrad) return sig * (1.0f - sig);
    if constexpr (FN == kNatSwishGrad) return sig * (1.0f + x * (1.0f - sig));
    return 0.0f;
}

template <int DT, int FN>
__device__ __forceinline__ uint32_t eval_native(uint32_t x) {
    return Sfu<DT>::pack(native_scalar<FN>(Sfu<DT>::lo(x)), native_scalar<FN>(Sfu<DT>::hi(x)));
}

}  // namespace fpt
