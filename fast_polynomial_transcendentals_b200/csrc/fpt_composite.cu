// FP16 composite element-wise operators around the degree-3 forward programs: forward with a saved derivative,
// fused forward + gradient, hybrid SFU / polynomial lane routing, and the plain product used by their backward.
// They read x once and write two arrays, or mix the two arithmetic pipes inside one 16-byte vector.
#include <cuda_fp16.h>

#include "fpt_programs.h"
#include "fpt_stream.cuh"

namespace fpt {
namespace {

constexpr int kDT = kFp16;
using P = Pk<kDT>;

// compile-time description of the three functions: shapes of the D3 forward and the D4 derivative programs
template <int FN> struct Fn;
template <> struct Fn<FPT_FN_SIGMOID> { static constexpr int fwd = kOddHalf, bwd = kEven, alg = kAlgSig; };
template <> struct Fn<FPT_FN_TANH> { static constexpr int fwd = kOdd, bwd = kEven, alg = kAlgTanh; };
template <> struct Fn<FPT_FN_SWISH> { static constexpr int fwd = kSwish, bwd = kOddHalf, alg = -1; };

// y = F_D3(x), dy = algebraic derivative from y (sigmoid: y(1-y); tanh: 1 - y^2)
template <int FN>
struct FwdDerivAlgOp {
    static constexpr int NIN = 1, NOUT = 2;
    ProgramWords f;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[2]) const {
        out[0] = eval_program<kDT, Fn<FN>::fwd, 3>(in[0], f);
        out[1] = eval_program<kDT, Fn<FN>::alg, 0>(out[0], f);
    }
};

// y = F_D3(x), dy = F'_D4(x): two polynomials on the same input
template <int FN>
struct FwdDerivPolyOp {
    static constexpr int NIN = 1, NOUT = 2;
    ProgramWords f, g;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[2]) const {
        out[0] = eval_program<kDT, Fn<FN>::fwd, 3>(in[0], f);
        out[1] = eval_program<kDT, Fn<FN>::bwd, 4>(in[0], g);
    }
};

// SiLU with one shared sigmoid: s = sigmoid_D3(x); y = x s; dy = s (1 + x (1 - s))
struct SwishSharedSigmoidOp {
    static constexpr int NIN = 1, NOUT = 2;
    ProgramWords sig;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[2]) const {
        const uint32_t s = eval_program<kDT, kOddHalf, 3>(in[0], sig);
        out[0] = P::mul(in[0], s);
        out[1] = P::mul(s, P::fma(in[0], P::sub(Consts<kDT>::one, s), Consts<kDT>::one));
    }
};

// in = (x, grad_out): y = F_D3(x), grad_in = grad_out * derivative (algebraic from y; SiLU: D4 polynomial of x)
template <int FN>
struct FusedFwdBwdOp {
    static constexpr int NIN = 2, NOUT = 2;
    ProgramWords f, g;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[2]) const {
        out[0] = eval_program<kDT, Fn<FN>::fwd, 3>(in[0], f);
        uint32_t d;
        if constexpr (FN == FPT_FN_SWISH) d = eval_program<kDT, Fn<FN>::bwd, 4>(in[0], g);
        else d = eval_program<kDT, Fn<FN>::alg, 0>(out[0], f);
        out[1] = P::mul(in[1], d);
    }
};

template <int DT>
struct MultiplyOp {
    static constexpr int NIN = 2, NOUT = 1;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<DT>::mul(in[0], in[1]);
    }
};

// ---- SFU lanes of the hybrid kernels: the toolkit's packed half intrinsics (ex2 / rcp / tanh on the XU pipe)
__device__ __forceinline__ __half2 as_h2(uint32_t w) { return *reinterpret_cast<__half2*>(&w); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// The transcendental itself comes from the intrinsic; the arithmetic around it uses this library's explicitly
// rounded packed operations, so that no multiply-add pair can be contracted behind the source's back.
template <int FN, bool BWD>
__device__ __forceinline__ uint32_t sfu_lane(uint32_t xw) {
    constexpr uint32_t one = Consts<kDT>::one;
    if constexpr (FN == FPT_FN_TANH) {
        const uint32_t y = as_u32(h2tanh_approx(as_h2(xw)));
        if constexpr (!BWD) return y;
        return P::sub(one, P::mul(y, y));
    } else {
        const uint32_t e = as_u32(h2exp(as_h2(xw ^ kSignMask)));
        const uint32_t s = as_u32(h2rcp(as_h2(P::add(one, e))));
        if constexpr (FN == FPT_FN_SIGMOID) {
            if constexpr (!BWD) return s;
            return P::mul(s, P::sub(one, s));
        } else {
            if constexpr (!BWD) return P::mul(xw, s);
            return P::mul(s, P::add(one, P::mul(xw, P::sub(one, s))));
        }
    }
}

// Of every four packed words (one 16-byte group) the first goes through the SFU, the other three through the
// polynomial.  Elements outside whole vectors (ragged tail, unaligned pointers) are all polynomial.
template <int FN, bool ROUTED>
struct HybridFwdOp {
    static constexpr int NIN = 1, NOUT = 1;
    static constexpr bool kIndexed = ROUTED;
    ProgramWords f;
    __device__ __forceinline__ void apply(const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        out[0] = eval_program<kDT, Fn<FN>::fwd, 3>(in[0], f);
    }
    __device__ __forceinline__ void apply_at(int word, const uint32_t (&in)[1], uint32_t (&out)[1]) const {
        if ((word & 3) == 0) out[0] = sfu_lane<FN, false>(in[0]);
        else apply(in, out);
    }
};

// in = (grad_out, x): grad_in = grad_out * derivative(x), derivative = D4 polynomial or its SFU twin
template <int FN, bool ROUTED>
struct HybridBwdOp {
    static constexpr int NIN = 2, NOUT = 1;
    static constexpr bool kIndexed = ROUTED;
    ProgramWords g;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = P::mul(in[0], eval_program<kDT, Fn<FN>::bwd, 4>(in[1], g));
    }
    __device__ __forceinline__ void apply_at(int word, const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        if ((word & 3) == 0) out[0] = P::mul(in[0], sfu_lane<FN, true>(in[1]));
        else apply(in, out);
    }
};

template <class F>
int dispatch_fn3(int function, F&& f) {
    switch (function) {
    case FPT_FN_SIGMOID: return f(IC<FPT_FN_SIGMOID>{});
    case FPT_FN_TANH: return f(IC<FPT_FN_TANH>{});
    case FPT_FN_SWISH: return f(IC<FPT_FN_SWISH>{});
    default: return FPT_ERR_BAD_ENUM;
    }
}

int words_for(int function, int direction, int degree, int shape, ProgramWords* w) {
    const ProgramRow* row = find_program(function, direction, degree, FPT_FP16, FPT_SRC_CURRENT);
    if (!row || row->shape != shape || row->degree != degree) return FPT_ERR_UNKNOWN_PROGRAM;
    *w = program_words(*row);
    return FPT_OK;
}

template <int FN>
int fwd_bwd_words(ProgramWords* f, ProgramWords* g) {
    if (int rc = words_for(FN, FPT_FWD, 3, Fn<FN>::fwd, f)) return rc;
    return words_for(FN, FPT_BWD, 4, Fn<FN>::bwd, g);
}

// the reference's rule for the routed kernels: whole 16-byte groups, at least 4096 packed words
bool hybrid_applies(int64_t n) { return (n % 8) == 0 && n / 2 >= 4096; }

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_fwd_deriv(void* y, void* dy, const void* x, int64_t n, int function, int variant,
                             fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!y || !dy || !x)) return FPT_ERR_NULL_POINTER;
    if (variant < FPT_DERIV_ALGEBRAIC || variant > FPT_DERIV_SHARED_SIGMOID) return FPT_ERR_BAD_ENUM;
    StreamArgs<1, 2> a{};
    a.in[0] = static_cast<const uint16_t*>(x);
    a.out[0] = static_cast<uint16_t*>(y);
    a.out[1] = static_cast<uint16_t*>(dy);
    if (variant == FPT_DERIV_SHARED_SIGMOID) {
        if (function != FPT_FN_SWISH) return FPT_ERR_UNKNOWN_PROGRAM;
        ProgramWords sig;
        if (int rc = words_for(FPT_FN_SIGMOID, FPT_FWD, 3, kOddHalf, &sig)) return rc;
        return launch_stream(SwishSharedSigmoidOp{sig}, a, n, stream);
    }
    if (variant == FPT_DERIV_ALGEBRAIC && function == FPT_FN_SWISH) return FPT_ERR_UNKNOWN_PROGRAM;
    return dispatch_fn3(function, [&](auto fn) {
        ProgramWords f, g;
        if (int rc = fwd_bwd_words<fn()>(&f, &g)) return rc;
        if (variant == FPT_DERIV_POLY) return launch_stream(FwdDerivPolyOp<fn()>{f, g}, a, n, stream);
        if constexpr (fn() != FPT_FN_SWISH) return launch_stream(FwdDerivAlgOp<fn()>{f}, a, n, stream);
        return int(FPT_ERR_UNKNOWN_PROGRAM);
    });
}

extern "C" int fpt_fused_fwd_bwd(void* y, void* grad_in, const void* x, const void* grad_out, int64_t n, int function,
                                 fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!y || !grad_in || !x || !grad_out)) return FPT_ERR_NULL_POINTER;
    StreamArgs<2, 2> a{};
    a.in[0] = static_cast<const uint16_t*>(x);
    a.in[1] = static_cast<const uint16_t*>(grad_out);
    a.out[0] = static_cast<uint16_t*>(y);
    a.out[1] = static_cast<uint16_t*>(grad_in);
    return dispatch_fn3(function, [&](auto fn) {
        ProgramWords f, g;
        if (int rc = fwd_bwd_words<fn()>(&f, &g)) return rc;
        return launch_stream(FusedFwdBwdOp<fn()>{f, g}, a, n, stream);
    });
}

extern "C" int fpt_multiply(void* out, const void* a_in, const void* b_in, int64_t n, int dtype, fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!out || !a_in || !b_in)) return FPT_ERR_NULL_POINTER;
    StreamArgs<2, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(a_in);
    a.in[1] = static_cast<const uint16_t*>(b_in);
    a.out[0] = static_cast<uint16_t*>(out);
    return dispatch_dtype(dtype, [&](auto dt) { return launch_stream(MultiplyOp<dt()>{}, a, n, stream); });
}

extern "C" int fpt_unary_hybrid(void* out, const void* in, int64_t n, int function, fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!out || !in)) return FPT_ERR_NULL_POINTER;
    StreamArgs<1, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(in);
    a.out[0] = static_cast<uint16_t*>(out);
    return dispatch_fn3(function, [&](auto fn) {
        ProgramWords f, g;
        if (int rc = fwd_bwd_words<fn()>(&f, &g)) return rc;
        if (!hybrid_applies(n)) return launch_stream(HybridFwdOp<fn(), false>{f}, a, n, stream);
        return launch_stream(HybridFwdOp<fn(), true>{f}, a, n, stream);
    });
}

extern "C" int fpt_binary_bwd_hybrid(void* grad_in, const void* grad_out, const void* x, int64_t n, int function,
                                     fpt_stream_t stream) {
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!grad_in || !grad_out || !x)) return FPT_ERR_NULL_POINTER;
    StreamArgs<2, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(grad_out);
    a.in[1] = static_cast<const uint16_t*>(x);
    a.out[0] = static_cast<uint16_t*>(grad_in);
    return dispatch_fn3(function, [&](auto fn) {
        ProgramWords f, g;
        if (int rc = fwd_bwd_words<fn()>(&f, &g)) return rc;
        if (!hybrid_applies(n)) return launch_stream(HybridBwdOp<fn(), false>{g}, a, n, stream);
        return launch_stream(HybridBwdOp<fn(), true>{g}, a, n, stream);
    });
}
