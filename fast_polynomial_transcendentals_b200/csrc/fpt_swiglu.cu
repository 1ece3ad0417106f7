// Fused SwiGLU element-wise operators: flat (routed experts, B4) and packed [gate | up] rows (dense FFN, B1),
// forward and backward.
#include "fpt_programs.h"
#include "fpt_stream.cuh"

namespace fpt {
namespace {

// out = swish(gate) * up        in[0] = gate, in[1] = up
template <int DT, int SHAPE, int DEG>
struct SwishMulOp {
    static constexpr int NIN = 2, NOUT = 1;
    ProgramWords p;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<DT>::mul(eval_program<DT, SHAPE, DEG>(in[0], p), in[1]);
    }
};

template <int DT>
struct NativeSwishMulOp {
    static constexpr int NIN = 2, NOUT = 1;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<DT>::mul(eval_native<DT, kNatSwish>(in[0]), in[1]);
    }
};

// in[0] = grad_out, in[1] = gate, in[2] = up;  out[0] = grad_gate, out[1] = grad_up
template <int DT, int FSHAPE, int DEG>
struct SwishMulBwdOp {
    static constexpr int NIN = 3, NOUT = 2;
    ProgramWords fwd, bwd;  // bwd is an ODD_HALF program of the same degree
    __device__ __forceinline__ void apply(const uint32_t (&in)[3], uint32_t (&out)[2]) const {
        using P = Pk<DT>;
        out[0] = P::mul(P::mul(in[0], in[2]), eval_program<DT, kOddHalf, DEG>(in[1], bwd));
        out[1] = P::mul(in[0], eval_program<DT, FSHAPE, DEG>(in[1], fwd));
    }
};

// One sigmoid evaluation shared by swish and its derivative:
// sig = sigmoid_d3(x); swish = x*sig; swish' = fma(swish, 1 - sig, sig)
template <int DT>
struct SwishMulBwdSharedSigmoidOp {
    static constexpr int NIN = 3, NOUT = 2;
    ProgramWords sigmoid;
    __device__ __forceinline__ void apply(const uint32_t (&in)[3], uint32_t (&out)[2]) const {
        using P = Pk<DT>;
        const uint32_t sig = eval_program<DT, kOddHalf, 3>(in[1], sigmoid);
        const uint32_t swish = P::mul(in[1], sig);
        const uint32_t deriv = P::fma(swish, P::sub(Consts<DT>::one, sig), sig);
        out[0] = P::mul(P::mul(in[0], in[2]), deriv);
        out[1] = P::mul(in[0], swish);
    }
};

template <int DT>
struct NativeSwishMulBwdOp {
    static constexpr int NIN = 3, NOUT = 2;
    __device__ __forceinline__ void apply(const uint32_t (&in)[3], uint32_t (&out)[2]) const {
        using P = Pk<DT>;
        const uint32_t dy = P::mul(in[0], in[2]);
        const float x0 = Sfu<DT>::lo(in[1]), x1 = Sfu<DT>::hi(in[1]);
        out[0] = Sfu<DT>::pack(Sfu<DT>::lo(dy) * native_scalar<kNatSwishGrad>(x0),
                               Sfu<DT>::hi(dy) * native_scalar<kNatSwishGrad>(x1));
        out[1] = P::mul(in[0], eval_native<DT, kNatSwish>(in[1]));
    }
};

constexpr unsigned kSwishShapes = (1u << kSwish) | (1u << kXmulHalf);

// ---- packed rows ----------------------------------------------------------------------------
// Thread layout inside a 256-thread block: 2^tx_shift column vectors x (256 >> tx_shift) rows, so that
// narrow rows still fill the block; R rows per thread are loaded before any is computed.

#ifndef FPT_PACKED_BLOCK
#define FPT_PACKED_BLOCK 256
#endif
constexpr int kPackedBlock = FPT_PACKED_BLOCK;

struct PackedArgs {
    const uint16_t* packed;    // [rows, 2*hidden]
    const uint16_t* grad_out;  // [rows, hidden] (backward only)
    uint16_t* out;             // forward: [rows, hidden]; backward: grad_packed [rows, 2*hidden]
    int64_t rows, hidden;
    int vecs_per_row, tx_shift;
};

template <class Op, int R, bool STREAM>
__global__ void __launch_bounds__(kPackedBlock) packed_fwd_kernel(const Op op, const PackedArgs a) {
    // grid.x walks along a row (column tile fastest in launch order), grid.y over row groups, so that the
    // blocks resident at any moment cover a few long contiguous spans.  Index math stays 32-bit and free of
    // divisions: with two loads per thread every extra instruction costs memory-level parallelism.
    const int tx = threadIdx.x & ((1 << a.tx_shift) - 1);
    const int ty = threadIdx.x >> a.tx_shift;
    const int rows_per_block = kPackedBlock >> a.tx_shift;
    const int col = (int(blockIdx.x) << a.tx_shift) + tx;
    if (col >= a.vecs_per_row) return;
    const int64_t row_step = int64_t(gridDim.y) * rows_per_block * R;
    // never unrolled: an unrolled grid-stride loop needs its trip count, i.e. a 64-bit division per thread
#pragma unroll 1
    for (int64_t row0 = int64_t(blockIdx.y) * rows_per_block * R + ty; row0 < a.rows; row0 += row_step) {
        Vec<4> g[R], u[R];
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int64_t row = row0 + int64_t(i) * rows_per_block;
            if (row < a.rows) {
                const Vec<4>* base = reinterpret_cast<const Vec<4>*>(a.packed + row * 2 * a.hidden);
                g[i] = load_vec<4, STREAM>(base + col);
                u[i] = load_vec<4, STREAM>(base + a.vecs_per_row + col);
            }
        }
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int64_t row = row0 + int64_t(i) * rows_per_block;
            if (row < a.rows) {
                Vec<4> r;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t in[2] = {g[i].w[w], u[i].w[w]};
                    uint32_t o[1];
                    op.apply(in, o);
                    r.w[w] = o[0];
                }
                store_vec<4, STREAM>(reinterpret_cast<Vec<4>*>(a.out + row * a.hidden) + col, r);
            }
        }
    }
}

template <class Op, int R, bool STREAM>
__global__ void __launch_bounds__(kPackedBlock) packed_bwd_kernel(const Op op, const PackedArgs a) {
    // grid.x walks along a row (column tile fastest in launch order), grid.y over row groups, so that the
    // blocks resident at any moment cover a few long contiguous spans.  Index math stays 32-bit and free of
    // divisions: with two loads per thread every extra instruction costs memory-level parallelism.
    const int tx = threadIdx.x & ((1 << a.tx_shift) - 1);
    const int ty = threadIdx.x >> a.tx_shift;
    const int rows_per_block = kPackedBlock >> a.tx_shift;
    const int col = (int(blockIdx.x) << a.tx_shift) + tx;
    if (col >= a.vecs_per_row) return;
    const int64_t row_step = int64_t(gridDim.y) * rows_per_block * R;
    // never unrolled: an unrolled grid-stride loop needs its trip count, i.e. a 64-bit division per thread
#pragma unroll 1
    for (int64_t row0 = int64_t(blockIdx.y) * rows_per_block * R + ty; row0 < a.rows; row0 += row_step) {
        Vec<4> go[R], g[R], u[R];
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int64_t row = row0 + int64_t(i) * rows_per_block;
            if (row < a.rows) {
                const Vec<4>* base = reinterpret_cast<const Vec<4>*>(a.packed + row * 2 * a.hidden);
                go[i] = load_vec<4, STREAM>(reinterpret_cast<const Vec<4>*>(a.grad_out + row * a.hidden) + col);
                g[i] = load_vec<4, STREAM>(base + col);
                u[i] = load_vec<4, STREAM>(base + a.vecs_per_row + col);
            }
        }
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int64_t row = row0 + int64_t(i) * rows_per_block;
            if (row < a.rows) {
                Vec<4> gg, gu;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t in[3] = {go[i].w[w], g[i].w[w], u[i].w[w]};
                    uint32_t o[2];
                    op.apply(in, o);
                    gg.w[w] = o[0];
                    gu.w[w] = o[1];
                }
                Vec<4>* base = reinterpret_cast<Vec<4>*>(a.out + row * 2 * a.hidden);
                store_vec<4, STREAM>(base + col, gg);
                store_vec<4, STREAM>(base + a.vecs_per_row + col, gu);
            }
        }
    }
}

// Any hidden size / alignment: one element per thread step.
template <class Op, bool BWD>
__global__ void __launch_bounds__(kBlock) packed_element_kernel(const Op op, const PackedArgs a) {
    const int64_t total = a.rows * a.hidden;
#pragma unroll 1
    for (int64_t e = int64_t(blockIdx.x) * kBlock + threadIdx.x; e < total; e += int64_t(gridDim.x) * kBlock) {
        const int64_t row = e / a.hidden, col = e - row * a.hidden;
        const uint32_t g = uint32_t(a.packed[row * 2 * a.hidden + col]) * 0x00010001u;
        const uint32_t u = uint32_t(a.packed[row * 2 * a.hidden + a.hidden + col]) * 0x00010001u;
        if constexpr (BWD) {
            const uint32_t in[3] = {uint32_t(a.grad_out[e]) * 0x00010001u, g, u};
            uint32_t o[2];
            op.apply(in, o);
            a.out[row * 2 * a.hidden + col] = uint16_t(o[0]);
            a.out[row * 2 * a.hidden + a.hidden + col] = uint16_t(o[1]);
        } else {
            const uint32_t in[2] = {g, u};
            uint32_t o[1];
            op.apply(in, o);
            a.out[e] = uint16_t(o[0]);
        }
    }
}

// One row per thread: like the flat kernels, two 128-bit loads in flight per thread and many short
// blocks measured best (B1 shape, 16384 x 14336: 4 rows per thread 6.85 TB/s).
constexpr int kPackedRows = 1;
#ifndef FPT_PACKED_ROWS_BWD
#define FPT_PACKED_ROWS_BWD 2
#endif
constexpr int kPackedRowsBwd = FPT_PACKED_ROWS_BWD;   // rows per thread and pass in the backward: two measured 0.6 % (16384 x 14336) to 2-3 % (131072 x 1408) faster than one

template <bool BWD, class Op>
int launch_packed(const Op& op, PackedArgs a, cudaStream_t stream) {
    if (a.rows == 0 || a.hidden == 0) return FPT_OK;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    const Tuning t = tuning();
    uintptr_t align = reinterpret_cast<uintptr_t>(a.packed) | reinterpret_cast<uintptr_t>(a.out) |
                      reinterpret_cast<uintptr_t>(a.grad_out);
    if (align & 1u) return FPT_ERR_MISALIGNED;
    if ((a.hidden % 8) != 0 || (align & 15u)) {
        int64_t grid = (a.rows * a.hidden + kBlock - 1) / kBlock;
        const int64_t cap = int64_t(dev.sm_count) * 32;
        if (grid > cap) grid = cap;
        packed_element_kernel<Op, BWD><<<unsigned(grid), kBlock, 0, stream>>>(op, a);
        return cuda_status(cudaGetLastError());
    }
    const int64_t vpr = a.hidden / 8;
    if (vpr > 0x7fffffff / 2) return FPT_ERR_BAD_SIZE;
    a.vecs_per_row = int(vpr);
    int shift = 0;
    while ((1 << shift) < kPackedBlock && (1 << shift) < a.vecs_per_row) ++shift;
    a.tx_shift = shift;
    const int rows_per_block = (kPackedBlock >> shift) * (BWD ? kPackedRowsBwd : kPackedRows);
    int64_t row_groups = (a.rows + rows_per_block - 1) / rows_per_block;
    const int64_t col_tiles = (vpr + (1 << shift) - 1) >> shift;
    if (t.blocks_per_sm > 0) {
        const int64_t cap = (int64_t(dev.sm_count) * t.blocks_per_sm + col_tiles - 1) / col_tiles;
        if (row_groups > cap) row_groups = cap;
    }
    if (row_groups > 65535) row_groups = 65535;  // grid.y limit; the kernel strides over the remaining rows
    const int64_t bytes = a.rows * a.hidden * 2 * (BWD ? 5 : 3);
    const bool streaming = t.streaming < 0 ? bytes > dev.l2_bytes : t.streaming != 0;
    const dim3 grid{unsigned(col_tiles), unsigned(row_groups), 1u};
    if constexpr (BWD) {
        if (streaming) packed_bwd_kernel<Op, kPackedRowsBwd, true><<<grid, kPackedBlock, 0, stream>>>(op, a);
        else packed_bwd_kernel<Op, kPackedRowsBwd, false><<<grid, kPackedBlock, 0, stream>>>(op, a);
    } else {
        if (streaming) packed_fwd_kernel<Op, kPackedRows, true><<<grid, kPackedBlock, 0, stream>>>(op, a);
        else packed_fwd_kernel<Op, kPackedRows, false><<<grid, kPackedBlock, 0, stream>>>(op, a);
    }
    return cuda_status(cudaGetLastError());
}

int check_enums(int dtype, int source) {
    if (dtype != FPT_FP16 && dtype != FPT_BF16) return FPT_ERR_BAD_ENUM;
    if (source != FPT_SRC_CURRENT && source != FPT_SRC_SOLLYA) return FPT_ERR_BAD_ENUM;
    return FPT_OK;
}

// Runs `f(op)` with the forward SwiGLU operator selected by (degree, dtype, source).
template <class F>
int with_swish_mul_op(int degree, int dtype, int source, F&& f) {
    if (degree == 0) return dispatch_dtype(dtype, [&](auto dt) { return f(NativeSwishMulOp<dt()>{}); });
    const ProgramRow* row = find_program(FPT_FN_SWISH, FPT_FWD, degree, dtype, source);
    if (!row) return FPT_ERR_UNKNOWN_PROGRAM;
    const ProgramWords words = program_words(*row);
    return dispatch_dtype(dtype, [&](auto dt) {
        return dispatch_shape_degree<kSwishShapes>(row->shape, row->degree, [&](auto sh, auto dg) {
            return f(SwishMulOp<dt(), sh(), dg()>{words});
        });
    });
}

template <class F>
int with_swish_mul_bwd_op(int degree, int dtype, int source, F&& f) {
    if (degree == 0) return dispatch_dtype(dtype, [&](auto dt) { return f(NativeSwishMulBwdOp<dt()>{}); });
    if (degree == 3 && dtype == FPT_BF16 && source == FPT_SRC_CURRENT) {
        const ProgramRow* sig = find_program(FPT_FN_SIGMOID, FPT_FWD, 3, dtype, source);
        if (!sig) return FPT_ERR_UNKNOWN_PROGRAM;
        return f(SwishMulBwdSharedSigmoidOp<kBf16>{program_words(*sig)});
    }
    const ProgramRow* fwd = find_program(FPT_FN_SWISH, FPT_FWD, degree, dtype, source);
    const ProgramRow* bwd = find_program(FPT_FN_SWISH, FPT_BWD, degree, dtype, source);
    if (!fwd || !bwd || bwd->shape != kOddHalf) return FPT_ERR_UNKNOWN_PROGRAM;
    const ProgramWords fw = program_words(*fwd), bw = program_words(*bwd);
    return dispatch_dtype(dtype, [&](auto dt) {
        return dispatch_shape_degree<kSwishShapes>(fwd->shape, fwd->degree, [&](auto sh, auto dg) {
            return f(SwishMulBwdOp<dt(), sh(), dg()>{fw, bw});
        });
    });
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_swish_mul(void* out, const void* gate, const void* up, int64_t n, int degree, int dtype,
                             int source, fpt_stream_t stream) {
    if (int rc = check_enums(dtype, source)) return rc;
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!out || !gate || !up)) return FPT_ERR_NULL_POINTER;
    StreamArgs<2, 1> a{};
    a.in[0] = static_cast<const uint16_t*>(gate);
    a.in[1] = static_cast<const uint16_t*>(up);
    a.out[0] = static_cast<uint16_t*>(out);
    return with_swish_mul_op(degree, dtype, source, [&](auto op) { return launch_stream(op, a, n, stream); });
}

extern "C" int fpt_swish_mul_bwd(void* grad_gate, void* grad_up, const void* grad_out, const void* gate,
                                 const void* up, int64_t n, int degree, int dtype, int source, fpt_stream_t stream) {
    if (int rc = check_enums(dtype, source)) return rc;
    if (n < 0) return FPT_ERR_BAD_SIZE;
    if (n > 0 && (!grad_gate || !grad_up || !grad_out || !gate || !up)) return FPT_ERR_NULL_POINTER;
    StreamArgs<3, 2> a{};
    a.in[0] = static_cast<const uint16_t*>(grad_out);
    a.in[1] = static_cast<const uint16_t*>(gate);
    a.in[2] = static_cast<const uint16_t*>(up);
    a.out[0] = static_cast<uint16_t*>(grad_gate);
    a.out[1] = static_cast<uint16_t*>(grad_up);
    return with_swish_mul_bwd_op(degree, dtype, source, [&](auto op) { return launch_stream(op, a, n, stream); });
}

extern "C" int fpt_swish_mul_packed(void* out, const void* packed, int64_t rows, int64_t hidden, int degree,
                                    int dtype, int source, fpt_stream_t stream) {
    if (int rc = check_enums(dtype, source)) return rc;
    if (rows < 0 || hidden < 0) return FPT_ERR_BAD_SIZE;
    if (rows > 0 && hidden > 0 && (!out || !packed)) return FPT_ERR_NULL_POINTER;
    PackedArgs a{};
    a.packed = static_cast<const uint16_t*>(packed);
    a.out = static_cast<uint16_t*>(out);
    a.rows = rows;
    a.hidden = hidden;
    return with_swish_mul_op(degree, dtype, source, [&](auto op) { return launch_packed<false>(op, a, stream); });
}

extern "C" int fpt_swish_mul_packed_bwd(void* grad_packed, const void* grad_out, const void* packed, int64_t rows,
                                        int64_t hidden, int degree, int dtype, int source, fpt_stream_t stream) {
    if (int rc = check_enums(dtype, source)) return rc;
    if (rows < 0 || hidden < 0) return FPT_ERR_BAD_SIZE;
    if (rows > 0 && hidden > 0 && (!grad_packed || !grad_out || !packed)) return FPT_ERR_NULL_POINTER;
    PackedArgs a{};
    a.packed = static_cast<const uint16_t*>(packed);
    a.grad_out = static_cast<const uint16_t*>(grad_out);
    a.out = static_cast<uint16_t*>(grad_packed);
    a.rows = rows;
    a.hidden = hidden;
    return with_swish_mul_bwd_op(degree, dtype, source, [&](auto op) { return launch_packed<true>(op, a, stream); });
}
