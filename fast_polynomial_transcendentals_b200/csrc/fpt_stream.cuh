// HBM-streaming element-wise kernel skeleton for sm_100a.
//
// One skeleton moves the bytes for every flat 16-bit element-wise operator of the
// library (unary activations, gradient products, SwiGLU, B3 sigmoid, fractional
// exp2): NIN input arrays and NOUT output arrays of the same length, processed in
// per-thread vectors of 128 or 256 bits.  Each thread issues UNROLL independent
// vector loads per input before it computes; the default grid is one block per
// tile (persistent grids of SM count x resident blocks measured 3-12 % slower on
// B200 and remain available through the "blocks_per_sm" tuning key).
// Above the L2 size the loads and stores carry streaming (evict-first) hints;
// below it they use the read-only path and plain stores so that back-to-back
// launches stay L2 resident.  A ragged tail (length not a multiple of the vector
// width) is finished by the last block with 16-bit accesses inside the same
// launch; misaligned pointers take the all-scalar kernel.
#pragma once

#include <cstdint>
#include <type_traits>
#include <cuda_runtime.h>

#include "fpt_common.h"

namespace fpt {

constexpr int kBlock = 256;  // fixed-shape kernels (packed rows, sin/cos, RoPE, scalar fallbacks)

template <int WORDS>
struct alignas(WORDS * 4) Vec {
    uint32_t w[WORDS];
};

template <int WORDS, bool STREAM>
__device__ __forceinline__ Vec<WORDS> load_vec(const void* p) {
    Vec<WORDS> v;
    if constexpr (WORDS == 4) {
        if constexpr (STREAM)
            asm volatile("ld.global.cs.v4.b32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
        else
            asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
    } else {
        if constexpr (STREAM)
            asm volatile("ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                           "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
        else
            asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                           "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    }
    return v;
}

template <int WORDS, bool STREAM>
__device__ __forceinline__ void store_vec(void* p, const Vec<WORDS>& v) {
    if constexpr (WORDS == 4) {
        if constexpr (STREAM)
            asm volatile("st.global.cs.v4.b32 [%0], {%1,%2,%3,%4};"
                         :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
        else
            asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};"
                         :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
    } else {
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]),
                        "r"(v.w[6]), "r"(v.w[7]) : "memory");
    }
}

template <int NIN, int NOUT>
struct StreamArgs {
    const uint16_t* in[NIN];
    uint16_t* out[NOUT];
    int64_t n_vec;   // whole vectors
    int64_t n_elem;  // all elements (tail = n_elem - n_vec * elements per vector)
};

// Op contract:  static constexpr int NIN, NOUT;
//               __device__ void apply(const uint32_t (&in)[NIN], uint32_t (&out)[NOUT]) const;   (two lanes per word)
// An Op with `static constexpr bool kIndexed = true` is instead called, inside whole vectors, as
//               apply_at(word, in, out)   word = index of the packed word within its vector (16-byte groups of four),
// which lets it treat the lanes of a group differently; tails and unaligned arrays still go through apply().
template <class Op, class = void>
struct op_indexed : std::false_type {};
template <class Op>
struct op_indexed<Op, std::void_t<decltype(Op::kIndexed)>> : std::integral_constant<bool, Op::kIndexed> {};

template <class Op, int WORDS, int UNROLL, bool STREAM, int BLOCK>
__global__ void __launch_bounds__(BLOCK) stream_kernel(const Op op, const StreamArgs<Op::NIN, Op::NOUT> a) {
    constexpr int NIN = Op::NIN, NOUT = Op::NOUT;
    constexpr int block = BLOCK;
    constexpr int64_t kTile = int64_t(block) * UNROLL;
    const int64_t stride = int64_t(gridDim.x) * kTile;
    // never unrolled: an unrolled grid-stride loop needs its trip count, i.e. a 64-bit division per thread
#pragma unroll 1
    for (int64_t tile = int64_t(blockIdx.x) * kTile; tile < a.n_vec; tile += stride) {
        const int64_t first = tile + threadIdx.x;
        Vec<WORDS> v[NIN][UNROLL];
        const bool full = tile + kTile <= a.n_vec;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t idx = first + int64_t(u) * block;
            if (full || idx < a.n_vec) {
#pragma unroll
                for (int i = 0; i < NIN; ++i)
                    v[i][u] = load_vec<WORDS, STREAM>(reinterpret_cast<const Vec<WORDS>*>(a.in[i]) + idx);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t idx = first + int64_t(u) * block;
            if (full || idx < a.n_vec) {
                Vec<WORDS> r[NOUT];
#pragma unroll
                for (int w = 0; w < WORDS; ++w) {
                    uint32_t xi[NIN], yo[NOUT];
#pragma unroll
                    for (int i = 0; i < NIN; ++i) xi[i] = v[i][u].w[w];
                    if constexpr (op_indexed<Op>::value) op.apply_at(w, xi, yo);
                    else op.apply(xi, yo);
#pragma unroll
                    for (int o = 0; o < NOUT; ++o) r[o].w[w] = yo[o];
                }
#pragma unroll
                for (int o = 0; o < NOUT; ++o)
                    store_vec<WORDS, STREAM>(reinterpret_cast<Vec<WORDS>*>(a.out[o]) + idx, r[o]);
            }
        }
    }
    if (blockIdx.x == gridDim.x - 1) {  // ragged tail, one element per thread step
#pragma unroll 1
        for (int64_t e = a.n_vec * (WORDS * 2) + threadIdx.x; e < a.n_elem; e += block) {
            uint32_t xi[NIN], yo[NOUT];
#pragma unroll
            for (int i = 0; i < NIN; ++i) xi[i] = uint32_t(a.in[i][e]) * 0x00010001u;
            op.apply(xi, yo);
#pragma unroll
            for (int o = 0; o < NOUT; ++o) a.out[o][e] = uint16_t(yo[o]);
        }
    }
}

// All-scalar variant for pointers that are not 16-byte aligned.
template <class Op>
__global__ void __launch_bounds__(kBlock) element_kernel(const Op op, const StreamArgs<Op::NIN, Op::NOUT> a) {
    constexpr int NIN = Op::NIN, NOUT = Op::NOUT;
#pragma unroll 1
    for (int64_t e = int64_t(blockIdx.x) * kBlock + threadIdx.x; e < a.n_elem; e += int64_t(gridDim.x) * kBlock) {
        uint32_t xi[NIN], yo[NOUT];
#pragma unroll
        for (int i = 0; i < NIN; ++i) xi[i] = uint32_t(a.in[i][e]) * 0x00010001u;
        op.apply(xi, yo);
#pragma unroll
        for (int o = 0; o < NOUT; ++o) a.out[o][e] = uint16_t(yo[o]);
    }
}

template <class Op, int WORDS, int UNROLL, bool STREAM, int BLOCK>
static int launch_stream_config(const Op& op, const StreamArgs<Op::NIN, Op::NOUT>& a, const DeviceInfo& dev,
                                const Tuning& t, cudaStream_t stream) {
    auto kernel = stream_kernel<Op, WORDS, UNROLL, STREAM, BLOCK>;
    constexpr int block = BLOCK;
    const int64_t tiles = (a.n_vec + int64_t(block) * UNROLL - 1) / (int64_t(block) * UNROLL);
    int64_t grid = tiles > 0 ? tiles : 1;
    if (t.blocks_per_sm > 0) {
        const int64_t cap = int64_t(dev.sm_count) * t.blocks_per_sm;
        if (grid > cap) grid = cap;
    }
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    kernel<<<unsigned(grid), block, 0, stream>>>(op, a);
    return cuda_status(cudaGetLastError());
}

// Launch configuration, chosen by measurement on B200 (fp16 sigmoid at 2^28 elements and bf16
// SwiGLU at 1.8e8..2.3e8 elements, every combination of 128/256-bit vectors, 1..8 vectors per
// thread and persistent grids of 2..32 blocks per SM): the best is always one block per tile
// with two 128-bit loads in flight per thread -- 6.78 TB/s unary, 7.07 TB/s SwiGLU -- while
// persistent grids lose 3..12 %.  So UNROLL = 2 / NIN (at least 1) and no grid cap by default.
#ifndef FPT_STREAM_WORDS
#define FPT_STREAM_WORDS 4
#endif
#ifndef FPT_LOADS_IN_FLIGHT
#define FPT_LOADS_IN_FLIGHT 2
#endif
#define FPT_RESIDENT_WORDS FPT_STREAM_WORDS
// Threads per block: 256 while streaming from HBM; 128 for L2-resident sizes, where the finer blocks
// balance the last wave over the 148 SMs (graph-replayed sigmoid, 2^20 / 2^22 elements: 1.78 / 3.03 us
// against 1.97 / 3.34 us with 256 threads).
#ifndef FPT_STREAM_BLOCK
#define FPT_STREAM_BLOCK 256
#endif
#ifndef FPT_RESIDENT_BLOCK
#define FPT_RESIDENT_BLOCK 128
#endif
template <int NIN>
constexpr int stream_unroll() { return FPT_LOADS_IN_FLIGHT / NIN > 0 ? FPT_LOADS_IN_FLIGHT / NIN : 1; }

// `bytes touched > L2` selects the streaming regime (evict-first hints).
template <class Op>
static int launch_stream(const Op& op, StreamArgs<Op::NIN, Op::NOUT> a, int64_t n_elem, cudaStream_t stream) {
    if (n_elem <= 0) return FPT_OK;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    const Tuning t = tuning();
    a.n_elem = n_elem;
    uintptr_t align = 0;
    for (int i = 0; i < Op::NIN; ++i) align |= reinterpret_cast<uintptr_t>(a.in[i]);
    for (int o = 0; o < Op::NOUT; ++o) align |= reinterpret_cast<uintptr_t>(a.out[o]);
    if (align & 1u) return FPT_ERR_MISALIGNED;
    const int64_t bytes = n_elem * 2 * (Op::NIN + Op::NOUT);
    const bool streaming = t.streaming < 0 ? bytes > dev.l2_bytes : t.streaming != 0;
    constexpr uintptr_t kStreamAlign = FPT_STREAM_WORDS * 4 - 1, kResidentAlign = FPT_RESIDENT_WORDS * 4 - 1;
    if (align & (streaming ? kStreamAlign : kResidentAlign)) {
        if constexpr (FPT_STREAM_WORDS == 8 || FPT_RESIDENT_WORDS == 8) {
            if (!(align & 15u)) {  // 16-byte aligned but not 32: narrow vectors
                a.n_vec = n_elem / 8;
                return launch_stream_config<Op, 4, 2, false, FPT_RESIDENT_BLOCK>(op, a, dev, t, stream);
            }
        }
        a.n_vec = 0;
        int64_t grid = (n_elem + kBlock - 1) / kBlock;
        const int64_t cap = int64_t(dev.sm_count) * 32;
        if (grid > cap) grid = cap;
        element_kernel<Op><<<unsigned(grid), kBlock, 0, stream>>>(op, a);
        return cuda_status(cudaGetLastError());
    }
    if (streaming) {
        a.n_vec = n_elem / (FPT_STREAM_WORDS * 2);
        return launch_stream_config<Op, FPT_STREAM_WORDS, stream_unroll<Op::NIN>(), true, FPT_STREAM_BLOCK>(op, a, dev, t, stream);
    }
    a.n_vec = n_elem / (FPT_RESIDENT_WORDS * 2);
    return launch_stream_config<Op, FPT_RESIDENT_WORDS, stream_unroll<Op::NIN>(), false, FPT_RESIDENT_BLOCK>(op, a, dev, t, stream);
}

}  // namespace fpt
