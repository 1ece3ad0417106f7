// Paired sin/cos in fp32: fp32 angles [n] -> out [2, n] fp32 (cos plane, sin plane), eight polynomial variants and the
// SFU control, plus their repeated-evaluation probes.  12 bytes per angle, so the kernel is an HBM stream: four
// angles per 128-bit load, two loads in flight per thread, streaming cache hints.
#include <cstdint>
#include <cuda_runtime.h>

#include "fpt_common.h"

namespace fpt {
namespace {

constexpr int kBlockF32 = 256;
constexpr int kLoadsInFlight = 2;

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
__device__ __forceinline__ float add_rn(float a, float b) {
    float d;
    asm("add.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ float mul_rn(float a, float b) {
    float d;
    asm("mul.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ float round_to_integer(float a) {
    float d;
    asm("cvt.rni.f32.f32 %0, %1;" : "=f"(d) : "f"(a));
    return d;
}
__device__ __forceinline__ float xor_bits(float v, uint32_t sign) { return __uint_as_float(__float_as_uint(v) ^ sign); }

enum ReducerF32 : int { kQuarterCvt = 0, kCycle = 1, kQuarterMagic2 = 2, kHalfMagic2 = 3, kHalfMagic1 = 4 };
constexpr float kBiasF32 = 12582912.0f;   // 1.5 * 2^23: adding it leaves the rounded integer in the low mantissa bits

struct CoeffsF32 {
    float sin_c[4];   // lowest order first: sin = r (s0 + s1 r^2 + ...)
    float cos_c[4];   // cos = c0 + c1 r^2 + ...
};

template <int REDUCER, int NSIN, int NCOS>
struct PolyF32 {
    CoeffsF32 k;
    __device__ __forceinline__ void operator()(float angle, float& cos_v, float& sin_v) const {
        float r;
        uint32_t sin_sign, cos_sign;
        bool swap = false;
        if constexpr (REDUCER == kQuarterCvt || REDUCER == kQuarterMagic2) {
            uint32_t q;
            float qf;
            if constexpr (REDUCER == kQuarterCvt) {
                const int qi = __float2int_rn(mul_rn(angle, 0.63661977236758134308f));
                qf = float(qi);
                q = uint32_t(qi);
            } else {
                const float biased = fma_rn(angle, 0.63661977236758134308f, kBiasF32);
                qf = sub_rn(biased, kBiasF32);
                q = __float_as_uint(biased);
            }
            r = fma_rn(qf, -1.57079625129699707031f, angle);
            r = fma_rn(qf, -7.54978941586159635335e-08f, r);
            swap = (q & 1u) != 0u;
            sin_sign = (q & 2u) << 30;
            cos_sign = ((q + 1u) & 2u) << 30;
        } else if constexpr (REDUCER == kHalfMagic2 || REDUCER == kHalfMagic1) {
            const float biased = fma_rn(angle, 0.31830988618379067154f, kBiasF32);
            const float h = sub_rn(biased, kBiasF32);
            if constexpr (REDUCER == kHalfMagic2) {
                r = fma_rn(h, -3.141592502593994140625f, angle);
                r = fma_rn(h, -1.50995788317231927067e-07f, r);
            } else {
                r = fma_rn(h, -3.1415927410125732421875f, angle);
            }
            sin_sign = cos_sign = (__float_as_uint(biased) & 1u) << 31;
        } else {
            // work in turns and fold by symmetry into [0, 1/8]
            const float cycles = mul_rn(angle, 0.15915494309189533577f);
            const float wrapped = sub_rn(cycles, round_to_integer(cycles));
            sin_sign = __float_as_uint(wrapped) & 0x80000000u;
            float a = fabsf(wrapped);
            const bool outer = a > 0.25f;
            a = outer ? sub_rn(0.5f, a) : a;
            swap = a > 0.125f;
            a = swap ? sub_rn(0.25f, a) : a;
            r = a;
            cos_sign = uint32_t(outer) << 31;
        }
        const float r2 = mul_rn(r, r);
        float sp = fma_rn(k.sin_c[NSIN - 1], r2, k.sin_c[NSIN - 2]);
#pragma unroll
        for (int i = NSIN - 3; i >= 0; --i) sp = fma_rn(sp, r2, k.sin_c[i]);
        sp = mul_rn(r, sp);
        float cp = fma_rn(k.cos_c[NCOS - 1], r2, k.cos_c[NCOS - 2]);
#pragma unroll
        for (int i = NCOS - 3; i >= 0; --i) cp = fma_rn(cp, r2, k.cos_c[i]);
        sin_v = xor_bits(swap ? cp : sp, sin_sign);
        cos_v = xor_bits(swap ? sp : cp, cos_sign);
    }
};

struct NativeF32 {   // the SFU control: sin.approx / cos.approx
    __device__ __forceinline__ void operator()(float angle, float& cos_v, float& sin_v) const {
        __sincosf(angle, &sin_v, &cos_v);
    }
};

struct ArgsF32 {
    const float* angles;
    float* cos_out;
    float* sin_out;
    int64_t n;        // elements
    int64_t n_vec;    // whole groups of four (0 when a pointer is not 16-byte aligned)
    int iterations;
};

template <class Ev, bool COMPUTE>
__device__ __forceinline__ void eval_one(const Ev& ev, float angle, int iterations, float& c, float& s) {
    if constexpr (!COMPUTE) {
        ev(angle, c, s);
    } else {
        float cs = 0.0f, ss = 0.0f, probe = angle;
#pragma unroll 1
        for (int it = 0; it < iterations; ++it) {
            float ci, si;
            ev(probe, ci, si);
            cs = add_rn(cs, ci);
            ss = add_rn(ss, si);
            probe = fma_rn(probe, 0.999999940395355224609375f, 0.0001220703125f);
        }
        c = cs;
        s = ss;
    }
}

template <class Ev, bool COMPUTE>
__global__ void __launch_bounds__(kBlockF32) sincos_f32_kernel(const Ev ev, const ArgsF32 a) {
    constexpr int64_t kTile = int64_t(kBlockF32) * kLoadsInFlight;
    const int64_t stride = int64_t(gridDim.x) * kTile;
#pragma unroll 1
    for (int64_t tile = int64_t(blockIdx.x) * kTile; tile < a.n_vec; tile += stride) {
        float4 in[kLoadsInFlight];
#pragma unroll
        for (int u = 0; u < kLoadsInFlight; ++u) {
            const int64_t idx = tile + threadIdx.x + int64_t(u) * kBlockF32;
            if (idx < a.n_vec) in[u] = __ldcs(reinterpret_cast<const float4*>(a.angles) + idx);
        }
#pragma unroll
        for (int u = 0; u < kLoadsInFlight; ++u) {
            const int64_t idx = tile + threadIdx.x + int64_t(u) * kBlockF32;
            if (idx < a.n_vec) {
                float4 c, s;
                eval_one<Ev, COMPUTE>(ev, in[u].x, a.iterations, c.x, s.x);
                eval_one<Ev, COMPUTE>(ev, in[u].y, a.iterations, c.y, s.y);
                eval_one<Ev, COMPUTE>(ev, in[u].z, a.iterations, c.z, s.z);
                eval_one<Ev, COMPUTE>(ev, in[u].w, a.iterations, c.w, s.w);
                __stcs(reinterpret_cast<float4*>(a.cos_out) + idx, c);
                __stcs(reinterpret_cast<float4*>(a.sin_out) + idx, s);
            }
        }
    }
    // elements outside whole vectors (a ragged end, or everything when a pointer is not 16-byte aligned)
#pragma unroll 1
    for (int64_t e = a.n_vec * 4 + int64_t(blockIdx.x) * kBlockF32 + threadIdx.x; e < a.n;
         e += int64_t(gridDim.x) * kBlockF32) {
        float c, s;
        eval_one<Ev, COMPUTE>(ev, a.angles[e], a.iterations, c, s);
        a.cos_out[e] = c;
        a.sin_out[e] = s;
    }
}

template <class Ev>
int launch_f32(const Ev& ev, ArgsF32 a, cudaStream_t stream) {
    constexpr int64_t kTile = int64_t(kBlockF32) * kLoadsInFlight;
    int64_t grid = (a.n_vec + kTile - 1) / kTile;
    const int64_t tail_blocks = (a.n - a.n_vec * 4 + kBlockF32 - 1) / kBlockF32;
    if (grid < tail_blocks) grid = tail_blocks;
    if (grid < 1) grid = 1;
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    if (a.iterations > 0) sincos_f32_kernel<Ev, true><<<unsigned(grid), kBlockF32, 0, stream>>>(ev, a);
    else sincos_f32_kernel<Ev, false><<<unsigned(grid), kBlockF32, 0, stream>>>(ev, a);
    return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_sincos_f32(void* out, const void* angles, int64_t n, int variant, int iterations, fpt_stream_t stream) {
    if (n < 0 || iterations < 0) return FPT_ERR_BAD_SIZE;
    if (variant < FPT_SINCOS_F32_NATIVE || variant > FPT_SINCOS_F32_D7_D6) return FPT_ERR_BAD_ENUM;
    if (n == 0) return FPT_OK;
    if (!out || !angles) return FPT_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(out) & 3u) || (reinterpret_cast<uintptr_t>(angles) & 3u)) return FPT_ERR_MISALIGNED;
    ArgsF32 a{};
    a.angles = static_cast<const float*>(angles);
    a.cos_out = static_cast<float*>(out);
    a.sin_out = a.cos_out + n;
    a.n = n;
    a.iterations = iterations;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a.angles) | reinterpret_cast<uintptr_t>(a.cos_out) |
                           reinterpret_cast<uintptr_t>(a.sin_out)) & 15u) == 0;
    a.n_vec = aligned ? n / 4 : 0;
    switch (variant) {
    case FPT_SINCOS_F32_NATIVE:
        return launch_f32(NativeF32{}, a, stream);
    case FPT_SINCOS_F32_D3_D4:
        return launch_f32(PolyF32<kQuarterCvt, 2, 3>{{{0.99903142452239990234375f, -0.16034401953220367431640625f},
            {0.999990046024322509765625f, -0.4997082054615020751953125f, 0.0403986163437366485595703125f}}}, a, stream);
    case FPT_SINCOS_F32_D3_D4_CYCLE:
        return launch_f32(PolyF32<kCycle, 2, 3>{{{6.277099609375f, -39.77336883544921875f},
            {0.999990046024322509765625f, -19.7276897430419921875f, 62.96308135986328125f}}}, a, stream);
    case FPT_SINCOS_F32_D3_D4_MAGIC_BIAS:
        return launch_f32(PolyF32<kQuarterMagic2, 2, 3>{{{0.99903142452239990234375f, -0.16034401953220367431640625f},
            {0.999990046024322509765625f, -0.4997082054615020751953125f, 0.0403986163437366485595703125f}}}, a, stream);
    case FPT_SINCOS_F32_D5_D4_HALF_TURN_LS:
        return launch_f32(PolyF32<kHalfMagic2, 3, 3>{{{0.999771416187286376953125f, -0.16582702100276947021484375f,
            0.00757423602044582366943359375f}, {0.999579489231109619140625f, -0.4963922202587127685546875f,
            0.0372092612087726593017578125f}}}, a, stream);
    case FPT_SINCOS_F32_D5_D4_HALF_TURN_SOLLYA:
        return launch_f32(PolyF32<kHalfMagic2, 3, 3>{{{0.999696791172027587890625f, -0.1656731069087982177734375f,
            0.0075143859721720218658447265625f}, {0.9994032382965087890625f, -0.495580852031707763671875f,
            0.03679168224334716796875f}}}, a, stream);
    case FPT_SINCOS_F32_D5_D4_HALF_TURN_SOLLYA_FAST:
        return launch_f32(PolyF32<kHalfMagic1, 3, 3>{{{0.999696791172027587890625f, -0.1656731069087982177734375f,
            0.0075143859721720218658447265625f}, {0.9994032382965087890625f, -0.495580852031707763671875f,
            0.03679168224334716796875f}}}, a, stream);
    case FPT_SINCOS_F32_D5_D4:
        return launch_f32(PolyF32<kQuarterCvt, 3, 3>{{{0.9999962449073792f, -0.16661198437213898f, 0.008137642405927181f},
            {0.999993085861206f, -0.499763548374176f, 0.04051213711500168f}}}, a, stream);
    default:
        return launch_f32(PolyF32<kQuarterCvt, 4, 4>{{{1.0f, -0.1666664183139801f, 0.00833179522305727f,
            -0.00019484198128338903f}, {1.0f, -0.49999886751174927f, 0.041656624525785446f, -0.0013605882413685322f}}},
            a, stream);
    }
}
