// Paired sin/cos (fp32 angles -> packed fp16 / bf16 cos and sin planes), RoPE tables from Q0.32 phases and the
// fused RoPE rotation with transpose.
#include <atomic>
#include <cstring>
#include <mutex>

#include "fpt_programs.h"
#include "fpt_stream.cuh"

namespace fpt {
namespace {

// ---- fp32 range reduction; every step is one explicitly rounded instruction ------------------------

__device__ __forceinline__ float fma_rn(float a, float b, float c) {
    float d;
    asm("fma.rn.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float sub_rn(float a, float b) {
    float d;
    asm("sub.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ float mul_rn(float a, float b) {
    float d;
    asm("mul.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

enum Reducer : int { kQuarterTwoTerm = 0, kQuarterMagic = 1, kHalfMagic = 2 };
constexpr float kBias = 12582912.0f;

// Returns the residual; `q` receives the quadrant (quarter-turn reducers) or the lane sign bit (half turn).
template <int REDUCER>
__device__ __forceinline__ float reduce_angle(float angle, uint32_t& q) {
    if constexpr (REDUCER == kQuarterTwoTerm) {
        const int qi = __float2int_rn(mul_rn(angle, 0.63661977236758134308f));
        const float qf = float(qi);
        float r = fma_rn(qf, -1.57079625129699707031f, angle);
        r = fma_rn(qf, -7.54978941586159635335e-08f, r);
        q = uint32_t(qi) & 3u;
        return r;
    } else if constexpr (REDUCER == kQuarterMagic) {
        const float biased = fma_rn(angle, 0.63661977236758134308f, kBias);
        const float qf = sub_rn(biased, kBias);
        q = __float_as_uint(biased);
        return fma_rn(qf, -1.57079637050628662109375f, angle);
    } else {
        const float biased = fma_rn(angle, 0.31830988618379067154f, kBias);
        const float hf = sub_rn(biased, kBias);
        q = (__float_as_uint(biased) & 1u) << 15;
        return fma_rn(hf, -3.1415927410125732421875f, angle);
    }
}

struct SincosWords {
    uint32_t sin_c[4];  // lowest order first: sin = r*(s0 + s1 r^2 + ...)
    uint32_t cos_c[4];  // cos = c0 + c1 r^2 + ...
};

// Two angles -> packed cos and sin words (low lane = first angle).
template <int EVAL_DT, int OUT_DT, int REDUCER, int NSIN, int NCOS>
__device__ __forceinline__ void sincos_pair(float a0, float a1, const SincosWords& k, uint32_t& cos_w, uint32_t& sin_w) {
    using P = Pk<EVAL_DT>;
    uint32_t q0, q1;
    const float r0 = reduce_angle<REDUCER>(a0, q0);
    const float r1 = reduce_angle<REDUCER>(a1, q1);
    const uint32_t r = Sfu<EVAL_DT>::pack(r0, r1);
    const uint32_t r2 = P::mul(r, r);
    uint32_t s = P::fma(k.sin_c[NSIN - 1], r2, k.sin_c[NSIN - 2]);
#pragma unroll
    for (int i = NSIN - 3; i >= 0; --i) s = P::fma(s, r2, k.sin_c[i]);
    s = P::mul(r, s);
    uint32_t c = P::fma(k.cos_c[NCOS - 1], r2, k.cos_c[NCOS - 2]);
#pragma unroll
    for (int i = NCOS - 3; i >= 0; --i) c = P::fma(c, r2, k.cos_c[i]);
    if constexpr (REDUCER == kHalfMagic) {
        const uint32_t signs = q0 | (q1 << 16);
        s ^= signs;
        c ^= signs;
    } else {
        const uint32_t swap = ((0u - (q0 & 1u)) & 0x0000ffffu) | ((0u - (q1 & 1u)) & 0xffff0000u);
        const uint32_t exchanged = (s ^ c) & swap;
        const uint32_t sin_sign = ((q0 & 2u) << 14) | ((q1 & 2u) << 30);
        const uint32_t cos_sign = (((q0 + 1u) & 2u) << 14) | (((q1 + 1u) & 2u) << 30);
        s = s ^ exchanged ^ sin_sign;
        c = c ^ exchanged ^ cos_sign;
    }
    if constexpr (EVAL_DT != OUT_DT) {  // fp16 evaluation stored as bf16: widen exactly, round once
        s = Sfu<OUT_DT>::pack(Sfu<EVAL_DT>::lo(s), Sfu<EVAL_DT>::hi(s));
        c = Sfu<OUT_DT>::pack(Sfu<EVAL_DT>::lo(c), Sfu<EVAL_DT>::hi(c));
    }
    sin_w = s;
    cos_w = c;
}

template <int OUT_DT>
__device__ __forceinline__ void sincos_pair_native(float a0, float a1, uint32_t& cos_w, uint32_t& sin_w) {
    // range-reduced MUFU sin/cos, two special-function operations per angle
    cos_w = Sfu<OUT_DT>::pack(__cosf(a0), __cosf(a1));
    sin_w = Sfu<OUT_DT>::pack(__sinf(a0), __sinf(a1));
}

struct SincosArgs {
    const float* angles;
    uint16_t* cos_out;
    uint16_t* sin_out;
    int64_t n;
    int iterations;  // 0: plain; >0: repeated-evaluation probe
};

// Ev contract: static constexpr int OUT_DT; __device__ void pair(float, float, uint32_t& cos, uint32_t& sin) const
template <class Ev, bool COMPUTE, bool STREAM>
__global__ void __launch_bounds__(kBlock) sincos_kernel(const Ev ev, const SincosArgs a) {
    const int64_t n_vec = a.n / 8;  // 8 angles: two 16-byte loads, one 16-byte store per plane
    const int64_t i = int64_t(blockIdx.x) * kBlock + threadIdx.x;
    if (i < n_vec) {
        const Vec<4> lo = load_vec<4, STREAM>(reinterpret_cast<const Vec<4>*>(a.angles) + 2 * i);
        const Vec<4> hi = load_vec<4, STREAM>(reinterpret_cast<const Vec<4>*>(a.angles) + 2 * i + 1);
        float ang[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            ang[j] = __uint_as_float(lo.w[j]);
            ang[4 + j] = __uint_as_float(hi.w[j]);
        }
        Vec<4> c, s;
        if constexpr (!COMPUTE) {
#pragma unroll
            for (int j = 0; j < 4; ++j) ev.pair(ang[2 * j], ang[2 * j + 1], c.w[j], s.w[j]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) c.w[j] = s.w[j] = 0u;
#pragma unroll 1
            for (int it = 0; it < a.iterations; ++it) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t cw, sw;
                    ev.pair(ang[2 * j], ang[2 * j + 1], cw, sw);
                    c.w[j] = Pk<Ev::OUT_DT>::add(c.w[j], cw);
                    s.w[j] = Pk<Ev::OUT_DT>::add(s.w[j], sw);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ang[j] = fma_rn(ang[j], 0.999999940395355224609375f, 0.0001220703125f);
            }
        }
        store_vec<4, STREAM>(reinterpret_cast<Vec<4>*>(a.cos_out) + i, c);
        store_vec<4, STREAM>(reinterpret_cast<Vec<4>*>(a.sin_out) + i, s);
    }
    if (blockIdx.x == gridDim.x - 1) {  // ragged tail
#pragma unroll 1
        for (int64_t e = n_vec * 8 + threadIdx.x; e < a.n; e += kBlock) {
            float p = a.angles[e];
            uint32_t cw, sw;
            if constexpr (!COMPUTE) {
                ev.pair(p, p, cw, sw);
            } else {
                cw = sw = 0u;
                for (int it = 0; it < a.iterations; ++it) {
                    uint32_t c1, s1;
                    ev.pair(p, p, c1, s1);
                    cw = Pk<Ev::OUT_DT>::add(cw, c1);
                    sw = Pk<Ev::OUT_DT>::add(sw, s1);
                    p = fma_rn(p, 0.999999940395355224609375f, 0.0001220703125f);
                }
            }
            a.cos_out[e] = uint16_t(cw);
            a.sin_out[e] = uint16_t(sw);
        }
    }
}

// element-at-a-time variant for planes that are not 16-byte aligned (n not a multiple of 8)
template <class Ev, bool COMPUTE>
__global__ void __launch_bounds__(kBlock) sincos_element_kernel(const Ev ev, const SincosArgs a) {
#pragma unroll 1
    for (int64_t e = int64_t(blockIdx.x) * kBlock + threadIdx.x; e < a.n; e += int64_t(gridDim.x) * kBlock) {
        float p = a.angles[e];
        uint32_t cw, sw;
        if constexpr (!COMPUTE) {
            ev.pair(p, p, cw, sw);
        } else {
            cw = sw = 0u;
            for (int it = 0; it < a.iterations; ++it) {
                uint32_t c1, s1;
                ev.pair(p, p, c1, s1);
                cw = Pk<Ev::OUT_DT>::add(cw, c1);
                sw = Pk<Ev::OUT_DT>::add(sw, s1);
                p = fma_rn(p, 0.999999940395355224609375f, 0.0001220703125f);
            }
        }
        a.cos_out[e] = uint16_t(cw);
        a.sin_out[e] = uint16_t(sw);
    }
}

template <int EVAL_DT, int OUT_DT_, int REDUCER, int NSIN, int NCOS>
struct PolyEv {
    static constexpr int OUT_DT = OUT_DT_;
    SincosWords k;
    __device__ __forceinline__ void pair(float a0, float a1, uint32_t& c, uint32_t& s) const {
        sincos_pair<EVAL_DT, OUT_DT_, REDUCER, NSIN, NCOS>(a0, a1, k, c, s);
    }
};
template <int OUT_DT_>
struct NativeEv {
    static constexpr int OUT_DT = OUT_DT_;
    __device__ __forceinline__ void pair(float a0, float a1, uint32_t& c, uint32_t& s) const {
        sincos_pair_native<OUT_DT_>(a0, a1, c, s);
    }
};

template <class Ev>
int launch_sincos(const Ev& ev, SincosArgs a, cudaStream_t stream) {
    if (a.n == 0) return FPT_OK;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    const uintptr_t align = reinterpret_cast<uintptr_t>(a.angles) | reinterpret_cast<uintptr_t>(a.cos_out) |
                            reinterpret_cast<uintptr_t>(a.sin_out);
    if ((reinterpret_cast<uintptr_t>(a.angles) & 3u) || (align & 1u)) return FPT_ERR_MISALIGNED;
    const bool compute = a.iterations > 0;
    if (align & 15u) {
        int64_t grid = (a.n + kBlock - 1) / kBlock;
        const int64_t cap = int64_t(dev.sm_count) * 32;
        if (grid > cap) grid = cap;
        if (compute) sincos_element_kernel<Ev, true><<<unsigned(grid), kBlock, 0, stream>>>(ev, a);
        else sincos_element_kernel<Ev, false><<<unsigned(grid), kBlock, 0, stream>>>(ev, a);
        return cuda_status(cudaGetLastError());
    }
    int64_t grid = (a.n / 8 + kBlock - 1) / kBlock;
    if (grid < 1) grid = 1;
    if (grid > 0x7fffffff) return FPT_ERR_BAD_SIZE;
    const bool streaming = tuning().streaming < 0 ? a.n * 8 > dev.l2_bytes : tuning().streaming != 0;
    if (compute) sincos_kernel<Ev, true, false><<<unsigned(grid), kBlock, 0, stream>>>(ev, a);
    else if (streaming) sincos_kernel<Ev, false, true><<<unsigned(grid), kBlock, 0, stream>>>(ev, a);
    else sincos_kernel<Ev, false, false><<<unsigned(grid), kBlock, 0, stream>>>(ev, a);
    return cuda_status(cudaGetLastError());
}

uint16_t f32_to_f16_bits(float x) {  // host: round to nearest even through the exact double path is not needed,
    // every coefficient below is exactly representable in its target format after this conversion
    uint32_t u;
    std::memcpy(&u, &x, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    int32_t e = int32_t((u >> 23) & 0xff) - 127 + 15;
    uint32_t m = u & 0x7fffffu;
    if (e <= 0) {
        if (e < -10) return uint16_t(sign);
        m |= 0x800000u;
        const int shift = 14 - e;
        uint32_t half = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return uint16_t(sign | half);
    }
    uint32_t half = (uint32_t(e) << 10) | (m >> 13);
    const uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
    return uint16_t(sign | half);
}
uint16_t f32_to_bf16_bits(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    return uint16_t((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

struct VariantDesc {
    int reducer, eval_dt, out_dt, n_sin, n_cos;
    float sin_c[4], cos_c[4];
};

// Coefficient sets of the packed evaluators (reference: sincos_kernels.cu:544-975), lowest order first.
const VariantDesc k_variants[FPT_SINCOS_VARIANT_COUNT] = {
    /* D3_D4_QUARTER_TURN_FP16 */ {kQuarterMagic, kFp16, kFp16, 2, 3, {0.9990234375f, -0.1602783203125f}, {1.0f, -0.499755859375f, 0.040435791015625f}},
    /* D3_D4_HALF_TURN_FP16 */ {kHalfMagic, kFp16, kFp16, 2, 3, {0.98876953125f, -0.14501953125f}, {0.99951171875f, -0.496337890625f, 0.037200927734375f}},
    /* D5_D4_HALF_TURN_FP16 */ {kHalfMagic, kFp16, kFp16, 3, 3, {0.99951171875f, -0.16552734375f, 0.0074920654296875f}, {0.99951171875f, -0.49560546875f, 0.036773681640625f}},
    /* D5_D6_HALF_TURN_FP16 */ {kHalfMagic, kFp16, kFp16, 3, 4, {0.99951171875f, -0.16552734375f, 0.0074920654296875f}, {1.0f, -0.499755859375f, 0.041412353515625f, -0.0012674331665039062f}},
    /* D7_D6_HALF_TURN_FP16 */ {kHalfMagic, kFp16, kFp16, 4, 4, {1.0f, -0.1666259765625f, 0.00829315185546875f, -0.00018227100372314453f}, {1.0f, -0.499755859375f, 0.041412353515625f, -0.0012674331665039062f}},
    /* D3_D4_BF16 */ {kQuarterTwoTerm, kBf16, kBf16, 2, 3, {0.99903142452239990234375f, -0.16034401953220367431640625f}, {0.999990046024322509765625f, -0.4997082054615020751953125f, 0.0403986163437366485595703125f}},
    /* D3_D4_QUARTER_TURN_BF16 */ {kQuarterMagic, kBf16, kBf16, 2, 3, {1.0f, -0.162109375f}, {1.0f, -0.5f, 0.041015625f}},
    /* D3_D4_HALF_TURN_BF16 */ {kHalfMagic, kBf16, kBf16, 2, 3, {0.98828125f, -0.1455078125f}, {1.0f, -0.49609375f, 0.037109375f}},
    /* D5_D6_HALF_TURN_BF16 */ {kHalfMagic, kBf16, kBf16, 3, 4, {1.0f, -0.166015625f, 0.007598876953125f}, {1.0f, -0.5f, 0.04150390625f, -0.00125885009765625f}},
    /* D5_D4_HALF_TURN_FP16_BF16 */ {kHalfMagic, kFp16, kBf16, 3, 3, {0.99951171875f, -0.16552734375f, 0.0074920654296875f}, {0.99951171875f, -0.49560546875f, 0.036773681640625f}},
};

SincosWords variant_words(const VariantDesc& v) {
    SincosWords w{};
    for (int i = 0; i < 4; ++i) {
        const uint16_t s = v.eval_dt == kFp16 ? f32_to_f16_bits(v.sin_c[i]) : f32_to_bf16_bits(v.sin_c[i]);
        const uint16_t c = v.eval_dt == kFp16 ? f32_to_f16_bits(v.cos_c[i]) : f32_to_bf16_bits(v.cos_c[i]);
        w.sin_c[i] = uint32_t(s) * 0x00010001u;
        w.cos_c[i] = uint32_t(c) * 0x00010001u;
    }
    return w;
}

// ---- RoPE ------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t short2_to_half2(int lo, int hi) {  // cvt.rn.f16.s16 on both lanes
    uint32_t d;
    asm("{.reg .f16 l, h; .reg .s16 a, b; cvt.s16.s32 a, %1; cvt.s16.s32 b, %2; cvt.rn.f16.s16 l, a; cvt.rn.f16.s16 h, b; mov.b32 %0, {l, h};}"
        : "=r"(d) : "r"(lo), "r"(hi));
    return d;
}

// Q0.32 phase = position * increment (mod 2^32).  Bits 15..30 read as a signed 16-bit residual r in [-1, 1)
// in quarter-turn units; sign = bit31 xor bit30.  sin: degree 5 odd, cos: degree 6 even, packed fp16.
__device__ __forceinline__ void rope_half_turn_d5_d6(uint32_t position, uint32_t inc0, uint32_t inc1, uint32_t& cos_w,
                                                     uint32_t& sin_w) {
    using P = Pk<kFp16>;
    const uint32_t p0 = position * inc0, p1 = position * inc1;
    const uint32_t r = P::mul(short2_to_half2(int(int16_t(p0 >> 15)), int(int16_t(p1 >> 15))), 0x02000200u);  // * 2^-15
    const uint32_t hi = __byte_perm(p0, p1, 0x7632);
    const uint32_t signs = (hi ^ (hi << 1)) & 0x80008000u;
    const uint32_t r2 = P::mul(r, r);
    uint32_t s = P::fma(0x2c9c2c9cu, r2, 0xb923b923u);  // 0.072021484375, -0.64208984375
    s = P::fma(s, r2, 0x3e483e48u);                     // 1.5703125
    s = P::mul(r, s);
    uint32_t c = P::fma(0xa4e3a4e3u, r2, 0x340a340au);  // -0.0190887451171875, 0.25244140625
    c = P::fma(c, r2, 0xbcefbcefu);                     // -1.2333984375
    c = P::fma(c, r2, 0x3c003c00u);                     // 1.0
    sin_w = s ^ signs;
    cos_w = c ^ signs;
}

// Q0.32 phase with a quarter-turn residual (sin degree 3, cos degree 4) and quadrant restore.
__device__ __forceinline__ void rope_quarter_turn_d3_d4(uint32_t position, uint32_t inc0, uint32_t inc1, uint32_t& cos_w,
                                                        uint32_t& sin_w) {
    using P = Pk<kFp16>;
    const uint32_t p0 = position * inc0, p1 = position * inc1;
    const uint32_t q0 = (p0 + 0x20000000u) >> 30, q1 = (p1 + 0x20000000u) >> 30;
    const int res0 = int(p0 - (q0 << 30)) >> 14, res1 = int(p1 - (q1 << 30)) >> 14;
    const uint32_t r = P::mul(short2_to_half2(int(int16_t(res0)), int(int16_t(res1))), 0x02000200u);
    const uint32_t r2 = P::mul(r, r);
    uint32_t s = P::fma(0xacf8acf8u, r2, 0x3a473a47u);  // -0.07763671875, 0.78466796875
    s = P::mul(r, s);
    uint32_t c = P::fma(0x23e123e1u, r2, 0xb4efb4efu);  // 0.01538848876953125, -0.308349609375
    c = P::fma(c, r2, 0x3c003c00u);
    const uint32_t swap = ((0u - (q0 & 1u)) & 0x0000ffffu) | ((0u - (q1 & 1u)) & 0xffff0000u);
    const uint32_t exchanged = (s ^ c) & swap;
    sin_w = s ^ exchanged ^ (((q0 & 2u) << 14) | ((q1 & 2u) << 30));
    cos_w = c ^ exchanged ^ ((((q0 + 1u) & 2u) << 14) | (((q1 + 1u) & 2u) << 30));
}

template <int KIND>
__device__ __forceinline__ void rope_pair(uint32_t position, uint32_t inc0, uint32_t inc1, float f0, float f1,
                                          uint32_t& c, uint32_t& s) {
    if constexpr (KIND == FPT_ROPE_HALF_TURN_D5_D6) rope_half_turn_d5_d6(position, inc0, inc1, c, s);
    else if constexpr (KIND == FPT_ROPE_QUARTER_TURN_D3_D4) rope_quarter_turn_d3_d4(position, inc0, inc1, c, s);
    else sincos_pair_native<kFp16>(float(position) * f0, float(position) * f1, c, s);
}

// table [2, S, F] fp16: cos plane then sin plane; params: int32 increments [F] (or fp32 frequencies for native)
template <int KIND>
__global__ void __launch_bounds__(kBlock) rope_table_kernel(const uint32_t* __restrict__ params, uint16_t* __restrict__ table,
                                                           int64_t seq, int64_t freq_count, int iterations) {
    const int64_t pairs = freq_count / 2;
    const int64_t total = seq * pairs;
    uint32_t* cos_plane = reinterpret_cast<uint32_t*>(table);
    uint32_t* sin_plane = reinterpret_cast<uint32_t*>(table + seq * freq_count);
#pragma unroll 1
    for (int64_t i = int64_t(blockIdx.x) * kBlock + threadIdx.x; i < total; i += int64_t(gridDim.x) * kBlock) {
        const int64_t pos = i / pairs, j = i - pos * pairs;
        const uint32_t a = params[2 * j], b = params[2 * j + 1];
        uint32_t c, s;
        if (iterations <= 0) {
            rope_pair<KIND>(uint32_t(pos), a, b, __uint_as_float(a), __uint_as_float(b), c, s);
        } else {  // repeated-evaluation probe: positions pos, pos+1, ... accumulated in fp16
            c = s = 0u;
            for (int it = 0; it < iterations; ++it) {
                uint32_t c1, s1;
                rope_pair<KIND>(uint32_t(pos) + uint32_t(it), a, b, __uint_as_float(a), __uint_as_float(b), c1, s1);
                c = Pk<kFp16>::add(c, c1);
                s = Pk<kFp16>::add(s, s1);
            }
        }
        cos_plane[pos * pairs + j] = c;
        sin_plane[pos * pairs + j] = s;
    }
}

// Look-up variant: the seven top phase bits (rounded) pick (sin, cos) from a 128-entry table held in shared memory,
// the signed remainder becomes an fp16 angle and one first-order step follows.
__device__ __forceinline__ void rope_lut_pair(uint32_t position, uint32_t inc0, uint32_t inc1, const uint32_t* lut,
                                              uint32_t& cos_w, uint32_t& sin_w) {
    using P = Pk<kFp16>;
    const uint32_t p0 = position * inc0, p1 = position * inc1;
    const uint32_t i0 = ((p0 + (1u << 24)) >> 25) & 127u, i1 = ((p1 + (1u << 24)) >> 25) & 127u;
    const float d0 = mul_rn(float(int(p0 - (i0 << 25))), 0x1.921fb6p-30f);   // 2 pi / 2^32 radians per phase unit
    const float d1 = mul_rn(float(int(p1 - (i1 << 25))), 0x1.921fb6p-30f);
    const uint32_t delta = Sfu<kFp16>::pack(d0, d1);
    const uint32_t b0 = lut[i0], b1 = lut[i1];
    const uint32_t sin_b = __byte_perm(b0, b1, 0x5410), cos_b = __byte_perm(b0, b1, 0x7632);
    sin_w = P::fma(delta, cos_b, sin_b);
    cos_w = P::fma(delta ^ kSignMask, sin_b, cos_b);
}

__global__ void __launch_bounds__(kBlock) rope_table_lut_kernel(const uint32_t* __restrict__ params,
                                                               const uint32_t* __restrict__ phase_table,
                                                               uint16_t* __restrict__ table, int64_t seq, int64_t freq_count,
                                                               int iterations) {
    __shared__ uint32_t lut[128];
    if (threadIdx.x < 128) lut[threadIdx.x] = phase_table[threadIdx.x];
    __syncthreads();
    const int64_t pairs = freq_count / 2;
    const int64_t total = seq * pairs;
    uint32_t* cos_plane = reinterpret_cast<uint32_t*>(table);
    uint32_t* sin_plane = reinterpret_cast<uint32_t*>(table + seq * freq_count);
#pragma unroll 1
    for (int64_t i = int64_t(blockIdx.x) * kBlock + threadIdx.x; i < total; i += int64_t(gridDim.x) * kBlock) {
        const int64_t pos = i / pairs, j = i - pos * pairs;
        const uint32_t a = params[2 * j], b = params[2 * j + 1];
        uint32_t c, s;
        if (iterations <= 0) {
            rope_lut_pair(uint32_t(pos), a, b, lut, c, s);
        } else {
            c = s = 0u;
            for (int it = 0; it < iterations; ++it) {
                uint32_t c1, s1;
                rope_lut_pair(uint32_t(pos) + uint32_t(it), a, b, lut, c1, s1);
                c = Pk<kFp16>::add(c, c1);
                s = Pk<kFp16>::add(s, s1);
            }
        }
        cos_plane[pos * pairs + j] = c;
        sin_plane[pos * pairs + j] = s;
    }
}

// 8 halves = 4 interleaved (even, odd) pairs; cos/sin words hold pairs (0,1) and (2,3).
template <bool IO_BF16>
__device__ __forceinline__ Vec<4> rotate_chunk(Vec<4> v, uint32_t cos_lo, uint32_t sin_lo, uint32_t cos_hi, uint32_t sin_hi) {
    using P = Pk<kFp16>;
    if constexpr (IO_BF16) {
#pragma unroll
        for (int w = 0; w < 4; ++w) v.w[w] = Sfu<kFp16>::pack(Sfu<kBf16>::lo(v.w[w]), Sfu<kBf16>::hi(v.w[w]));
    }
    const uint32_t even_lo = __byte_perm(v.w[0], v.w[1], 0x5410), odd_lo = __byte_perm(v.w[0], v.w[1], 0x7632);
    const uint32_t even_hi = __byte_perm(v.w[2], v.w[3], 0x5410), odd_hi = __byte_perm(v.w[2], v.w[3], 0x7632);
    const uint32_t re_lo = P::fma(sin_lo ^ kSignMask, odd_lo, P::mul(cos_lo, even_lo));
    const uint32_t ro_lo = P::fma(sin_lo, even_lo, P::mul(cos_lo, odd_lo));
    const uint32_t re_hi = P::fma(sin_hi ^ kSignMask, odd_hi, P::mul(cos_hi, even_hi));
    const uint32_t ro_hi = P::fma(sin_hi, even_hi, P::mul(cos_hi, odd_hi));
    Vec<4> r;
    r.w[0] = __byte_perm(re_lo, ro_lo, 0x5410);
    r.w[1] = __byte_perm(re_lo, ro_lo, 0x7632);
    r.w[2] = __byte_perm(re_hi, ro_hi, 0x5410);
    r.w[3] = __byte_perm(re_hi, ro_hi, 0x7632);
    if constexpr (IO_BF16) {
#pragma unroll
        for (int w = 0; w < 4; ++w) r.w[w] = Sfu<kBf16>::pack(Sfu<kFp16>::lo(r.w[w]), Sfu<kFp16>::hi(r.w[w]));
    }
    return r;
}

struct RopeApplyArgs {
    const uint16_t *q, *k;
    uint16_t *q_out, *k_out;
    const uint32_t* params;  // increments (int32), frequencies (fp32) or a cached table [2,S,D/2] fp16
    int64_t batch, seq, q_heads, k_heads;
    int chunks;              // head_dim / 8
    int pos_per_block;       // 256 / chunks_pow2
    int chunk_shift;
    int heads_per_block;     // heads of Q and of K one block rotates (grid.z walks the head groups)
};

// Block = (2^chunk_shift chunks) x (positions); each thread owns one (position, 8-wide chunk): it evaluates
// the four (cos, sin) pairs once and rotates that chunk for every Q head and every K head, writing [B,H,S,D].
template <int KIND, bool IO_BF16>
__global__ void __launch_bounds__(kBlock) rope_apply_kernel(const RopeApplyArgs a) {
    const int chunk = threadIdx.x & ((1 << a.chunk_shift) - 1);
    const int64_t pos = int64_t(blockIdx.x) * a.pos_per_block + (threadIdx.x >> a.chunk_shift);
    const int64_t b = blockIdx.y;
    if (chunk >= a.chunks || pos >= a.seq) return;
    uint32_t cos_lo, sin_lo, cos_hi, sin_hi;
    if constexpr (KIND == FPT_ROPE_CACHED) {
        const int64_t half_dim = int64_t(a.chunks) * 4;
        const uint2 c = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.params) + pos * half_dim + chunk * 4);
        const uint2 s = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.params) + (a.seq + pos) * half_dim + chunk * 4);
        cos_lo = c.x; cos_hi = c.y; sin_lo = s.x; sin_hi = s.y;
    } else {
        const uint4 inc = reinterpret_cast<const uint4*>(a.params)[chunk];
        rope_pair<KIND>(uint32_t(pos), inc.x, inc.y, __uint_as_float(inc.x), __uint_as_float(inc.y), cos_lo, sin_lo);
        rope_pair<KIND>(uint32_t(pos), inc.z, inc.w, __uint_as_float(inc.z), __uint_as_float(inc.w), cos_hi, sin_hi);
    }
    const int64_t token = b * a.seq + pos;
    {
        const Vec<4>* in = reinterpret_cast<const Vec<4>*>(a.q) + token * a.q_heads * a.chunks + chunk;
        Vec<4>* out = reinterpret_cast<Vec<4>*>(a.q_out) + (b * a.q_heads * a.seq + pos) * a.chunks + chunk;
        const int64_t out_step = a.seq * a.chunks;
        int64_t h = int64_t(blockIdx.z) * a.heads_per_block;
        const int64_t h_end = min(a.q_heads, h + a.heads_per_block);
        for (; h + 4 <= h_end; h += 4) {
            Vec<4> v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = load_vec<4, true>(in + (h + u) * a.chunks);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                store_vec<4, true>(out + (h + u) * out_step, rotate_chunk<IO_BF16>(v[u], cos_lo, sin_lo, cos_hi, sin_hi));
        }
        for (; h < h_end; ++h)
            store_vec<4, true>(out + h * out_step,
                               rotate_chunk<IO_BF16>(load_vec<4, true>(in + h * a.chunks), cos_lo, sin_lo, cos_hi, sin_hi));
    }
    {
        const Vec<4>* in = reinterpret_cast<const Vec<4>*>(a.k) + token * a.k_heads * a.chunks + chunk;
        Vec<4>* out = reinterpret_cast<Vec<4>*>(a.k_out) + (b * a.k_heads * a.seq + pos) * a.chunks + chunk;
        const int64_t out_step = a.seq * a.chunks;
        int64_t h = int64_t(blockIdx.z) * a.heads_per_block;
        const int64_t h_end = min(a.k_heads, h + a.heads_per_block);
        for (; h + 4 <= h_end; h += 4) {
            Vec<4> v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = load_vec<4, true>(in + (h + u) * a.chunks);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                store_vec<4, true>(out + (h + u) * out_step, rotate_chunk<IO_BF16>(v[u], cos_lo, sin_lo, cos_hi, sin_hi));
        }
        for (; h < h_end; ++h)
            store_vec<4, true>(out + h * out_step,
                               rotate_chunk<IO_BF16>(load_vec<4, true>(in + h * a.chunks), cos_lo, sin_lo, cos_hi, sin_hi));
    }
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_sincos(void* out, const void* angles, int64_t n, int variant, int iterations, fpt_stream_t stream) {
    if (n < 0 || iterations < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!out || !angles)) return FPT_ERR_NULL_POINTER;
    SincosArgs a{};
    a.angles = static_cast<const float*>(angles);
    a.cos_out = static_cast<uint16_t*>(out);
    a.sin_out = a.cos_out + n;
    a.n = n;
    a.iterations = iterations;
    if (variant == FPT_SINCOS_NATIVE_FP16) return launch_sincos(NativeEv<kFp16>{}, a, stream);
    if (variant == FPT_SINCOS_NATIVE_BF16) return launch_sincos(NativeEv<kBf16>{}, a, stream);
    if (variant < 0 || variant >= FPT_SINCOS_VARIANT_COUNT) return FPT_ERR_BAD_ENUM;
    const VariantDesc& v = k_variants[variant];
    const SincosWords w = variant_words(v);
    switch (variant) {
    case FPT_SINCOS_D3_D4_QUARTER_TURN_FP16: return launch_sincos(PolyEv<kFp16, kFp16, kQuarterMagic, 2, 3>{w}, a, stream);
    case FPT_SINCOS_D3_D4_HALF_TURN_FP16: return launch_sincos(PolyEv<kFp16, kFp16, kHalfMagic, 2, 3>{w}, a, stream);
    case FPT_SINCOS_D5_D4_HALF_TURN_FP16: return launch_sincos(PolyEv<kFp16, kFp16, kHalfMagic, 3, 3>{w}, a, stream);
    case FPT_SINCOS_D5_D6_HALF_TURN_FP16: return launch_sincos(PolyEv<kFp16, kFp16, kHalfMagic, 3, 4>{w}, a, stream);
    case FPT_SINCOS_D7_D6_HALF_TURN_FP16: return launch_sincos(PolyEv<kFp16, kFp16, kHalfMagic, 4, 4>{w}, a, stream);
    case FPT_SINCOS_D3_D4_BF16: return launch_sincos(PolyEv<kBf16, kBf16, kQuarterTwoTerm, 2, 3>{w}, a, stream);
    case FPT_SINCOS_D3_D4_QUARTER_TURN_BF16: return launch_sincos(PolyEv<kBf16, kBf16, kQuarterMagic, 2, 3>{w}, a, stream);
    case FPT_SINCOS_D3_D4_HALF_TURN_BF16: return launch_sincos(PolyEv<kBf16, kBf16, kHalfMagic, 2, 3>{w}, a, stream);
    case FPT_SINCOS_D5_D6_HALF_TURN_BF16: return launch_sincos(PolyEv<kBf16, kBf16, kHalfMagic, 3, 4>{w}, a, stream);
    case FPT_SINCOS_D5_D4_HALF_TURN_FP16_BF16: return launch_sincos(PolyEv<kFp16, kBf16, kHalfMagic, 3, 3>{w}, a, stream);
    default: return FPT_ERR_BAD_ENUM;
    }
}

extern "C" int fpt_rope_table(void* table, const void* params, int64_t seq, int64_t freq_count, int kind,
                              int iterations, fpt_stream_t stream) {
    if (seq < 0 || freq_count < 0 || iterations < 0) return FPT_ERR_BAD_SIZE;
    if (freq_count % 2) return FPT_ERR_BAD_SIZE;
    if (seq > 0x7fffffff) return FPT_ERR_BAD_SIZE;
    if (seq * freq_count == 0) return FPT_OK;
    if (!table || !params) return FPT_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(table) & 3u) || (reinterpret_cast<uintptr_t>(params) & 3u)) return FPT_ERR_MISALIGNED;
    if ((seq * freq_count) % 2) return FPT_ERR_BAD_SIZE;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    int64_t grid = (seq * (freq_count / 2) + kBlock - 1) / kBlock;
    const int64_t cap = int64_t(dev.sm_count) * 64;
    if (grid > cap) grid = cap;
    const uint32_t* p = static_cast<const uint32_t*>(params);
    uint16_t* t = static_cast<uint16_t*>(table);
    switch (kind) {
    case FPT_ROPE_HALF_TURN_D5_D6: rope_table_kernel<FPT_ROPE_HALF_TURN_D5_D6><<<unsigned(grid), kBlock, 0, stream>>>(p, t, seq, freq_count, iterations); break;
    case FPT_ROPE_QUARTER_TURN_D3_D4: rope_table_kernel<FPT_ROPE_QUARTER_TURN_D3_D4><<<unsigned(grid), kBlock, 0, stream>>>(p, t, seq, freq_count, iterations); break;
    case FPT_ROPE_NATIVE: rope_table_kernel<FPT_ROPE_NATIVE><<<unsigned(grid), kBlock, 0, stream>>>(p, t, seq, freq_count, iterations); break;
    default: return FPT_ERR_BAD_ENUM;
    }
    return cuda_status(cudaGetLastError());
}

extern "C" int fpt_rope_table_lut(void* table, const void* phase_increments, const void* phase_table, int64_t seq,
                                  int64_t freq_count, int iterations, fpt_stream_t stream) {
    if (seq < 0 || freq_count < 0 || iterations < 0) return FPT_ERR_BAD_SIZE;
    if (freq_count % 2) return FPT_ERR_BAD_SIZE;
    if (seq > 0x7fffffff) return FPT_ERR_BAD_SIZE;
    if (seq * freq_count == 0) return FPT_OK;
    if (!table || !phase_increments || !phase_table) return FPT_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(table) & 3u) || (reinterpret_cast<uintptr_t>(phase_increments) & 3u) ||
        (reinterpret_cast<uintptr_t>(phase_table) & 3u))
        return FPT_ERR_MISALIGNED;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    int64_t grid = (seq * (freq_count / 2) + kBlock - 1) / kBlock;
    const int64_t cap = int64_t(dev.sm_count) * 64;
    if (grid > cap) grid = cap;
    rope_table_lut_kernel<<<unsigned(grid), kBlock, 0, stream>>>(static_cast<const uint32_t*>(phase_increments),
                                                                static_cast<const uint32_t*>(phase_table),
                                                                static_cast<uint16_t*>(table), seq, freq_count, iterations);
    return cuda_status(cudaGetLastError());
}

// Argument checks of the fused rotation, separate from the launch so that an entry point which enqueues other work
// first can run them before anything is enqueued.  *empty is set when there is nothing to do.
static int rope_apply_validate(const void* q_out, const void* k_out, const void* q, const void* k, const void* params,
                               int64_t batch, int64_t seq, int64_t q_heads, int64_t k_heads, int64_t head_dim, int dtype,
                               bool* empty) {
    *empty = false;
    if (batch < 0 || seq < 0 || q_heads < 0 || k_heads < 0 || head_dim < 0) return FPT_ERR_BAD_SIZE;
    if (head_dim % 8 || head_dim > 2048) return FPT_ERR_BAD_SIZE;
    if (batch > 65535 || seq > 0x7fffffff) return FPT_ERR_BAD_SIZE;
    if (dtype != FPT_FP16 && dtype != FPT_BF16) return FPT_ERR_BAD_ENUM;
    if (batch * seq * head_dim == 0 || q_heads + k_heads == 0) {
        *empty = true;
        return FPT_OK;
    }
    if (!q_out || !k_out || !q || !k || !params) return FPT_ERR_NULL_POINTER;
    const uintptr_t align = reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_out) |
                            reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                            reinterpret_cast<uintptr_t>(params);
    if (align & 15u) return FPT_ERR_MISALIGNED;
    const int64_t most_heads = q_heads > k_heads ? q_heads : k_heads;
    const int tuned = fpt::tuning_rope_heads_per_block();
    const int64_t heads_per_block = tuned > 0 && tuned < most_heads ? tuned : most_heads;
    if ((most_heads + heads_per_block - 1) / heads_per_block > 65535) return FPT_ERR_BAD_SIZE;
    return FPT_OK;
}

extern "C" int fpt_rope_apply(void* q_out, void* k_out, const void* q, const void* k, const void* params, int64_t batch,
                              int64_t seq, int64_t q_heads, int64_t k_heads, int64_t head_dim, int kind, int dtype,
                              fpt_stream_t stream) {
    bool empty = false;
    if (int rc = rope_apply_validate(q_out, k_out, q, k, params, batch, seq, q_heads, k_heads, head_dim, dtype, &empty))
        return rc;
    if (empty) return FPT_OK;
    if (kind != FPT_ROPE_HALF_TURN_D5_D6 && kind != FPT_ROPE_NATIVE && kind != FPT_ROPE_CACHED) return FPT_ERR_BAD_ENUM;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    RopeApplyArgs a{};
    a.q = static_cast<const uint16_t*>(q);
    a.k = static_cast<const uint16_t*>(k);
    a.q_out = static_cast<uint16_t*>(q_out);
    a.k_out = static_cast<uint16_t*>(k_out);
    a.params = static_cast<const uint32_t*>(params);
    a.batch = batch; a.seq = seq; a.q_heads = q_heads; a.k_heads = k_heads;
    a.chunks = int(head_dim / 8);
    int shift = 0;
    while ((1 << shift) < a.chunks) ++shift;
    a.chunk_shift = shift;
    a.pos_per_block = kBlock >> shift;
    if (a.pos_per_block < 1) return FPT_ERR_BAD_SIZE;
    const int64_t most_heads = q_heads > k_heads ? q_heads : k_heads;
    const int tuned = fpt::tuning_rope_heads_per_block();
    a.heads_per_block = int(tuned > 0 && tuned < most_heads ? tuned : most_heads);
    const int64_t head_groups = (most_heads + a.heads_per_block - 1) / a.heads_per_block;
    if (head_groups > 65535) return FPT_ERR_BAD_SIZE;
    const dim3 grid{unsigned((seq + a.pos_per_block - 1) / a.pos_per_block), unsigned(batch), unsigned(head_groups)};
#define FPT_ROPE_CASE(K)                                                                              \
    case K:                                                                                           \
        if (dtype == FPT_BF16) rope_apply_kernel<K, true><<<grid, kBlock, 0, stream>>>(a);            \
        else rope_apply_kernel<K, false><<<grid, kBlock, 0, stream>>>(a);                             \
        break;
    switch (kind) {
        FPT_ROPE_CASE(FPT_ROPE_HALF_TURN_D5_D6)
        FPT_ROPE_CASE(FPT_ROPE_NATIVE)
        FPT_ROPE_CASE(FPT_ROPE_CACHED)
    default: return FPT_ERR_BAD_ENUM;
    }
#undef FPT_ROPE_CASE
    return cuda_status(cudaGetLastError());
}

// ---- fused RoPE from a cached table, for callers that cannot allocate device memory ----------------------
//
// The cached-table rotation needs a [2, seq, head_dim/2] fp16 table between its two kernels.  Code that runs
// where device allocation is off limits -- a plugin called inside a serving loop whose host owns every byte of
// device memory, a real-time path that may not take the allocator lock, a library user without a CUDA allocator
// of its own -- cannot provide that buffer.  For them the table lives in the fixed array below, which every GPU
// that loads this library holds until the process exits.
namespace fpt {
namespace {

constexpr int64_t kStaticRopeTableHalves = int64_t(1) << 21;  // 4 MiB: seq * head_dim <= 2^21, e.g. 16384 x 128

static __device__ __align__(256) uint16_t g_rope_table_scratch[kStaticRopeTableHalves];

// The array's name is a host-side handle, not a device address: the address has to be asked for, once per
// device, with that device current.
struct StaticTableAddress {
    std::atomic<int> ready{0};
    void* ptr = nullptr;
};
StaticTableAddress g_static_table[64];
std::mutex g_static_table_mutex;

int static_rope_table_address(void** out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ? FPT_ERR_NO_DEVICE : int(e);
    if (device < 0 || device >= 64) return FPT_ERR_NO_DEVICE;
    StaticTableAddress& slot = g_static_table[device];
    if (!slot.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_static_table_mutex);
        if (!slot.ready.load(std::memory_order_relaxed)) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_rope_table_scratch);
            if (e != cudaSuccess) return int(e);
            if (!p) return FPT_ERR_NULL_POINTER;
            slot.ptr = p;
            slot.ready.store(1, std::memory_order_release);
        }
    }
    *out = slot.ptr;
    return FPT_OK;
}

}  // namespace
}  // namespace fpt

extern "C" int64_t fpt_rope_static_table_capacity(void) { return fpt::kStaticRopeTableHalves; }

extern "C" int fpt_rope_apply_static_table(void* q_out, void* k_out, const void* q, const void* k,
                                           const void* phase_increments, int64_t batch, int64_t seq, int64_t q_heads,
                                           int64_t k_heads, int64_t head_dim, int table_kind, int dtype,
                                           fpt_stream_t stream) {
    if (table_kind != FPT_ROPE_HALF_TURN_D5_D6 && table_kind != FPT_ROPE_QUARTER_TURN_D3_D4) return FPT_ERR_BAD_ENUM;
    // every check of the two steps comes first: an error return means that nothing was enqueued and the shared table
    // still holds what the last successful call left in it
    bool empty = false;
    alignas(16) static const char aligned_stand_in = 0;      // stands for the table until its address is known
    if (int rc = rope_apply_validate(q_out, k_out, q, k, &aligned_stand_in, batch, seq, q_heads, k_heads, head_dim, dtype,
                                     &empty))
        return rc;
    if (seq > 0 && head_dim > 0 && seq > fpt::kStaticRopeTableHalves / head_dim) return FPT_ERR_SCRATCH_TOO_SMALL;
    if (empty) return FPT_OK;
    if (!phase_increments) return FPT_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(phase_increments) & 3u) return FPT_ERR_MISALIGNED;
    fpt::DeviceInfo dev;
    if (int rc = fpt::current_device_info(&dev)) return rc;
    void* table = nullptr;
    if (int rc = fpt::static_rope_table_address(&table)) return rc;
    // every entry of the [2, seq, head_dim/2] region used below is rewritten here, so nothing left over from an
    // earlier call is ever read
    if (int rc = fpt_rope_table(table, phase_increments, seq, head_dim / 2, table_kind, 0, stream)) return rc;
    return fpt_rope_apply(q_out, k_out, q, k, table, batch, seq, q_heads, k_heads, head_dim, FPT_ROPE_CACHED, dtype, stream);
}
