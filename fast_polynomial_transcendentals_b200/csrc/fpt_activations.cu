// Unary polynomial activations, their repeated-evaluation probes and gradient products.
#include "fpt_programs.h"
#include "fpt_stream.cuh"

namespace fpt {
namespace {

template <int DT, int SHAPE, int DEG>
struct UnaryOp {
    static constexpr int NIN = 1, NOUT = 1;
    ProgramWords p;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        out[0] = eval_program<DT, SHAPE, DEG>(in[0], p);
    }
};

template <int DT, int FN>
struct NativeUnaryOp {
    static constexpr int NIN = 1, NOUT = 1;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        if constexpr (FN == kNatTanh) out[0] = Sfu<DT>::tanh(in[0]);
        else out[0] = eval_native<DT, FN>(in[0]);
    }
};

template <int DT, int SHAPE, int DEG>
struct UnaryRepeatOp {
    static constexpr int NIN = 1, NOUT = 1;
    ProgramWords p;
    int repeats;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        uint32_t v = in[0];
#pragma unroll 1
        for (int r = 0; r < repeats; ++r) v = eval_program<DT, SHAPE, DEG>(v, p);
        out[0] = v;
    }
};

template <int DT, int FN>
struct NativeRepeatOp {
    static constexpr int NIN = 1, NOUT = 1;
    int repeats;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        uint32_t v = in[0];
#pragma unroll 1
        for (int r = 0; r < repeats; ++r) {
            if constexpr (FN == kNatTanh) v = Sfu<DT>::tanh(v);
            else v = eval_native<DT, FN>(v);
        }
        out[0] = v;
    }
};

// grad_in = grad_out * F(x)     in[0] = grad_out, in[1] = x
template <int DT, int SHAPE, int DEG>
struct GradMulOp {
    static constexpr int NIN = 2, NOUT = 1;
    ProgramWords p;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<DT>::mul(in[0], eval_program<DT, SHAPE, DEG>(in[1], p));
    }
};

template <int DT, int FN>
struct NativeGradMulOp {
    static constexpr int NIN = 2, NOUT = 1;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<DT>::mul(in[0], eval_native<DT, FN>(in[1]));
    }
};

constexpr unsigned kAllPolyShapes = (1u << kOddHalf) | (1u << kOdd) | (1u << kOddSat) | (1u << kSwish) |
                                    (1u << kXmulHalf) | (1u << kEven);
constexpr unsigned kGradShapes = (1u << kOddHalf) | (1u << kEven);

int native_fn(int function, int direction) {
    static const int fwd[] = {kNatSigmoid, kNatTanh, kNatSwish, kNatErf, kNatGelu};
    static const int bwd[] = {kNatSigmoidGrad, kNatTanhGrad, kNatSwishGrad, -1, kNatGeluGrad};
    if (function < 0 || function > FPT_FN_GELU) return -1;
    return direction == FPT_FWD ? fwd[function] : bwd[function];
}

template <class F>
int dispatch_native(int fn, F&& f) {
    switch (fn) {
    case kNatSigmoid: return f(IC<kNatSigmoid>{});
    case kNatTanh: return f(IC<kNatTanh>{});
    case kNatSwish: return f(IC<kNatSwish>{});
    case kNatSwishGrad: return f(IC<kNatSwishGrad>{});
    case kNatSigmoidGrad: return f(IC<kNatSigmoidGrad>{});
    case kNatTanhGrad: return f(IC<kNatTanhGrad>{});
    case kNatGelu: return f(IC<kNatGelu>{});
    case kNatGeluGrad: return f(IC<kNatGeluGrad>{});
    case kNatErf: return f(IC<kNatErf>{});
    default: return FPT_ERR_UNKNOWN_PROGRAM;
    }
}

int check_common(const void* a, const void* b, int64_t n, int dtype, int source) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!a || !b)) return FPT_ERR_NULL_POINTER;
    if (dtype != FPT_FP16 && dtype != FPT_BF16) return FPT_ERR_BAD_ENUM;
    if (source != FPT_SRC_CURRENT && source != FPT_SRC_SOLLYA) return FPT_ERR_BAD_ENUM;
    return FPT_OK;
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_unary_repeat(void* out, const void* in, int64_t n, int function, int direction, int degree,
                                int dtype, int source, int repeats, fpt_stream_t stream) {
    if (int rc = check_common(out, in, n, dtype, source)) return rc;
    if (repeats < 1) return FPT_ERR_BAD_SIZE;
    StreamArgs<1, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(in);
    a.out[0] = static_cast<uint16_t*>(out);
    if (degree == 0) {
        const int fn = native_fn(function, direction);
        return dispatch_dtype(dtype, [&](auto dt) {
            return dispatch_native(fn, [&](auto f) {
                if (repeats == 1) return launch_stream(NativeUnaryOp<dt(), f()>{}, a, n, stream);
                return launch_stream(NativeRepeatOp<dt(), f()>{repeats}, a, n, stream);
            });
        });
    }
    const ProgramRow* row = find_program(function, direction, degree, dtype, source);
    if (!row) return FPT_ERR_UNKNOWN_PROGRAM;
    const ProgramWords words = program_words(*row);
    return dispatch_dtype(dtype, [&](auto dt) {
        return dispatch_shape_degree<kAllPolyShapes>(row->shape, row->degree, [&](auto sh, auto dg) {
            if (repeats == 1) return launch_stream(UnaryOp<dt(), sh(), dg()>{words}, a, n, stream);
            return launch_stream(UnaryRepeatOp<dt(), sh(), dg()>{words, repeats}, a, n, stream);
        });
    });
}

extern "C" int fpt_unary(void* out, const void* in, int64_t n, int function, int direction, int degree, int dtype,
                         int source, fpt_stream_t stream) {
    return fpt_unary_repeat(out, in, n, function, direction, degree, dtype, source, 1, stream);
}

extern "C" int fpt_binary_bwd(void* grad_in, const void* grad_out, const void* x, int64_t n, int function,
                              int degree, int dtype, int source, fpt_stream_t stream) {
    if (int rc = check_common(grad_in, grad_out, n, dtype, source)) return rc;
    if (n > 0 && !x) return FPT_ERR_NULL_POINTER;
    StreamArgs<2, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(grad_out);
    a.in[1] = static_cast<const uint16_t*>(x);
    a.out[0] = static_cast<uint16_t*>(grad_in);
    if (degree == 0) {
        const int fn = native_fn(function, FPT_BWD);
        return dispatch_dtype(dtype, [&](auto dt) {
            return dispatch_native(fn, [&](auto f) { return launch_stream(NativeGradMulOp<dt(), f()>{}, a, n, stream); });
        });
    }
    const ProgramRow* row = find_program(function, FPT_BWD, degree, dtype, source);
    if (!row) return FPT_ERR_UNKNOWN_PROGRAM;
    const ProgramWords words = program_words(*row);
    return dispatch_dtype(dtype, [&](auto dt) {
        return dispatch_shape_degree<kGradShapes>(row->shape, row->degree, [&](auto sh, auto dg) {
            return launch_stream(GradMulOp<dt(), sh(), dg()>{words}, a, n, stream);
        });
    });
}

extern "C" int fpt_bwd_algebraic(void* grad_in, const void* grad_out, const void* y, int64_t n, int function,
                                 int dtype, fpt_stream_t stream) {
    if (int rc = check_common(grad_in, grad_out, n, dtype, FPT_SRC_CURRENT)) return rc;
    if (n > 0 && !y) return FPT_ERR_NULL_POINTER;
    if (function != FPT_FN_SIGMOID && function != FPT_FN_TANH) return FPT_ERR_UNKNOWN_PROGRAM;
    StreamArgs<2, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(grad_out);
    a.in[1] = static_cast<const uint16_t*>(y);
    a.out[0] = static_cast<uint16_t*>(grad_in);
    const ProgramWords none{};
    return dispatch_dtype(dtype, [&](auto dt) {
        if (function == FPT_FN_SIGMOID) return launch_stream(GradMulOp<dt(), kAlgSig, 0>{none}, a, n, stream);
        return launch_stream(GradMulOp<dt(), kAlgTanh, 0>{none}, a, n, stream);
    });
}
