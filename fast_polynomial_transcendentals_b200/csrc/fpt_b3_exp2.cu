// Isolated score-mod evaluators: the direct piecewise-cubic sigmoid of sigmoid attention (B3) and the
// fractional exp2 hinge, as flat element-wise kernels.
#include <type_traits>

#include "fpt_programs.h"
#include "fpt_scoremod.cuh"
#include "fpt_stream.cuh"

namespace fpt {
namespace {

// LATE: the evaluation order of the attention kernels (both rows on the FMA pipe, one select afterwards, no lower
// clamp, floor folded into the last multiply-add) instead of the deployed instruction order.
template <bool WITH_GRAD, bool LATE>
__device__ __forceinline__ uint32_t b3_eval(uint32_t x, const B3Words& k, uint32_t& grad) {
    if constexpr (WITH_GRAD) return LATE ? b3_direct_with_grad_select_late(x, k, grad) : b3_direct_with_grad(x, k, grad);
    else return LATE ? b3_direct_select_late(x, k) : b3_direct(x, k);
}

template <bool WITH_GRAD, bool LATE>
struct B3Op {
    static constexpr int NIN = 1, NOUT = WITH_GRAD ? 2 : 1;
    B3Words k;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[NOUT]) const {
        uint32_t g = 0;
        out[0] = b3_eval<WITH_GRAD, LATE>(in[0], k, g);
        if constexpr (WITH_GRAD) out[1] = g;
    }
};

// fp32 scores -> bf16 probabilities (the form in which the attention kernel meets the evaluator)
template <bool WITH_GRAD, bool LATE>
__global__ void __launch_bounds__(kBlock) b3_from_f32_kernel(const B3Words k, const float* __restrict__ scores,
                                                            uint16_t* __restrict__ prob, uint16_t* __restrict__ grad,
                                                            int64_t n) {
    const int64_t pairs = n / 2;
#pragma unroll 1
    for (int64_t i = int64_t(blockIdx.x) * kBlock + threadIdx.x; i < pairs; i += int64_t(gridDim.x) * kBlock) {
        const float2 s = reinterpret_cast<const float2*>(scores)[i];
        // the late-select order with a gradient converts as the attention backward does (no infinite lanes)
        const uint32_t x = (LATE && WITH_GRAD) ? Sfu<kBf16>::pack_satfinite(s.x, s.y) : Sfu<kBf16>::pack(s.x, s.y);
        uint32_t g = 0;
        reinterpret_cast<uint32_t*>(prob)[i] = b3_eval<WITH_GRAD, LATE>(x, k, g);
        if constexpr (WITH_GRAD) reinterpret_cast<uint32_t*>(grad)[i] = g;
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) {
        const uint32_t x = (LATE && WITH_GRAD) ? Sfu<kBf16>::pack_satfinite(scores[n - 1], scores[n - 1])
                                                : Sfu<kBf16>::pack(scores[n - 1], scores[n - 1]);
        uint32_t g = 0;
        const uint32_t p = b3_eval<WITH_GRAD, LATE>(x, k, g);
        prob[n - 1] = uint16_t(p);
        if constexpr (WITH_GRAD) grad[n - 1] = uint16_t(g);
    }
}

template <int VARIANT>  // 0 native MUFU ex2, 1 hinge
struct Exp2Op {
    static constexpr int NIN = 1, NOUT = 1;
    Exp2Words k;
    int repeats;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        uint32_t x = in[0], v = 0;
#pragma unroll 1
        for (int r = 0; r < repeats; ++r) {
            if constexpr (VARIANT == 0) v = Sfu<kFp16>::ex2(x);
            else v = exp2_hinge(x, k);
            x = Pk<kFp16>::fma(v, 0x38003800u, 0xb800b800u);  // back into [0, 1): v/2 - 1/2
        }
        out[0] = v;
    }
};

// fp32 2^a through the full-range software evaluators (cubic or two-piece line after floor reduction): the
// stand-alone form of what the attention kernel mixes with the special-function unit.  Four values per thread and step.
template <int KIND>
__global__ void __launch_bounds__(kBlock) exp2_full_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                              int64_t n) {
    const int64_t quads = n / 4;
#pragma unroll 1
    for (int64_t i = int64_t(blockIdx.x) * kBlock + threadIdx.x; i < quads; i += int64_t(gridDim.x) * kBlock) {
        const float4 a = reinterpret_cast<const float4*>(in)[i];
        float4 e;
        exp2_full_x2<KIND>(a.x, a.y, e.x, e.y);
        exp2_full_x2<KIND>(a.z, a.w, e.z, e.w);
        reinterpret_cast<float4*>(out)[i] = e;
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
        const int64_t i = quads * 4 + threadIdx.x;
        out[i] = exp2_full<KIND>(in[i]);
    }
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_b3_sigmoid_direct_variant(void* prob, void* grad, const void* scores, int64_t n, int scores_are_f32,
                                             int log2_n, int variant, fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!prob || !scores)) return FPT_ERR_NULL_POINTER;
    if (log2_n < 1 || log2_n > 24) return FPT_ERR_BAD_SIZE;
    if (variant != FPT_B3_DEPLOYED_ORDER && variant != FPT_B3_SELECT_LATE) return FPT_ERR_BAD_ENUM;
    const B3Words k = b3_words(log2_n);
    if (n == 0) return FPT_OK;
    auto run = [&](auto with_grad, auto late) -> int {
        constexpr bool G = decltype(with_grad)::value, L = decltype(late)::value;
        if (scores_are_f32) {
            DeviceInfo dev;
            if (int rc = current_device_info(&dev)) return rc;
            if ((reinterpret_cast<uintptr_t>(scores) & 7u) || (reinterpret_cast<uintptr_t>(prob) & 3u) ||
                (reinterpret_cast<uintptr_t>(grad) & 3u))
                return FPT_ERR_MISALIGNED;
            int64_t grid = (n / 2 + kBlock - 1) / kBlock;
            if (grid < 1) grid = 1;
            const int64_t cap = int64_t(dev.sm_count) * 64;
            if (grid > cap) grid = cap;
            b3_from_f32_kernel<G, L><<<unsigned(grid), kBlock, 0, stream>>>(
                k, static_cast<const float*>(scores), static_cast<uint16_t*>(prob), static_cast<uint16_t*>(grad), n);
            return cuda_status(cudaGetLastError());
        }
        StreamArgs<1, G ? 2 : 1> a{};
        a.in[0] = static_cast<const uint16_t*>(scores);
        a.out[0] = static_cast<uint16_t*>(prob);
        if constexpr (G) a.out[1] = static_cast<uint16_t*>(grad);
        return launch_stream(B3Op<G, L>{k}, a, n, stream);
    };
    const bool late = variant == FPT_B3_SELECT_LATE;
    if (grad) return late ? run(std::true_type{}, std::true_type{}) : run(std::true_type{}, std::false_type{});
    return late ? run(std::false_type{}, std::true_type{}) : run(std::false_type{}, std::false_type{});
}

extern "C" int fpt_b3_sigmoid_direct(void* prob, void* grad, const void* scores, int64_t n, int scores_are_f32,
                                     int log2_n, fpt_stream_t stream) {
    return fpt_b3_sigmoid_direct_variant(prob, grad, scores, n, scores_are_f32, log2_n, FPT_B3_DEPLOYED_ORDER, stream);
}

extern "C" int fpt_exp2_fraction(void* out, const void* in, int64_t n, int variant, int repeats, fpt_stream_t stream) {
    if (n < 0 || repeats < 1) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!out || !in)) return FPT_ERR_NULL_POINTER;
    if (variant < FPT_EXP2_NATIVE || variant > FPT_EXP2_HINGE_ENDPOINT) return FPT_ERR_BAD_ENUM;
    StreamArgs<1, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(in);
    a.out[0] = static_cast<uint16_t*>(out);
    if (variant == FPT_EXP2_NATIVE) return launch_stream(Exp2Op<0>{Exp2Words{}, repeats}, a, n, stream);
    return launch_stream(Exp2Op<1>{exp2_words(variant == FPT_EXP2_HINGE_ENDPOINT), repeats}, a, n, stream);
}

extern "C" int fpt_exp2_full_f32(void* out, const void* in, int64_t n, int variant, fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (variant < FPT_EXP2_FULL_D3 || variant > FPT_EXP2_FULL_PWL2_SAFE_F16) return FPT_ERR_BAD_ENUM;
    if (n == 0) return FPT_OK;
    if (!out || !in) return FPT_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return FPT_ERR_MISALIGNED;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    int64_t grid = (n / 4 + kBlock - 1) / kBlock;
    if (grid < 1) grid = 1;
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    const float* src = static_cast<const float*>(in);
    float* dst = static_cast<float*>(out);
    switch (variant) {
    case FPT_EXP2_FULL_D3: exp2_full_f32_kernel<kExp2FullD3><<<unsigned(grid), kBlock, 0, stream>>>(src, dst, n); break;
    case FPT_EXP2_FULL_PWL2: exp2_full_f32_kernel<kExp2FullPwl2><<<unsigned(grid), kBlock, 0, stream>>>(src, dst, n); break;
    case FPT_EXP2_FULL_D2_SAFE: exp2_full_f32_kernel<kExp2FullD2Safe><<<unsigned(grid), kBlock, 0, stream>>>(src, dst, n); break;
    default: exp2_full_f32_kernel<kExp2FullPwl2SafeF16><<<unsigned(grid), kBlock, 0, stream>>>(src, dst, n); break;
    }
    return cuda_status(cudaGetLastError());
}
