// Attention backward for sm_100a, same score-mods as the forward (soft-capped softmax, direct sigmoid, plain softmax).
//
// Two forms.  The single-pass form (attention_bwd_pipelined_kernel, further down: dK, dV and dQ in one kernel, 5 matrix
// products per tile pair, dQ accumulated in an fp32 buffer by reduce-add copies) and the two-pass form described here:
// two launches of one kernel template, each deterministic and free of atomics (S and dP are recomputed in both):
//   WHICH = 0  dQ:      one CTA per (batch, query head, 128 query rows), loops over key tiles
//                       S = Q K^T,  dP = dO V^T,  dS = f(S, dP),  dQ += dS K
//   WHICH = 1  dK, dV:  one CTA per (batch, kv head, 128 keys), loops over the query heads of its group and their
//                       query tiles;  S^T = K Q^T,  dP^T = V dO^T,  dV += P^T dO,  dK += dS^T Q
// Written once in terms of "fixed" tiles X, Y (loaded once) and "streamed" tiles U, W (2-stage ring):
//   S = X U^T and dP = Y W^T (both operands K-major from shared memory),
//   acc0 += dS U and (WHICH = 1) acc1 += P W, with P / dS read from tensor memory and U / W as MN-major operands.
// Roles: warp 0 TMA producer, warp 1 tcgen05.mma issuer (converged warp, elected lane), warps 4..11 score-mod warps: thread = one
// tensor-memory lane (row of the fixed tile), warps w and w+4 share a lane quarter and split the 128 columns in halves
// (the backward has no row reduction, so the split needs no exchange).
// Tensor memory: S is never overwritten (each score-mod warp writes its bf16 dS and P words over its own 64 columns of
// the dP tile), so the S product of the next step runs under the score-mod of the current one; dQ also double-buffers
// dP.  A pre-pass writes lse * log2(e) and delta = rowsum(dO * O) into a caller-provided workspace.
// Every mbarrier wait is bounded; on a timeout the CTA records where it stopped and unwinds.
#include <cstring>
#include <type_traits>

#include "fpt_common.h"
#include "fpt_programs.h"
#include "fpt_scoremod.cuh"
#include "fpt_sm100.cuh"

namespace fpt {
namespace {

using namespace sm100;

constexpr int kTile = 128;
constexpr int kDim = 128;
constexpr int kRing = 2;
constexpr uint32_t kPanelB = 128 * 128;        // bytes of one [128 rows x 64 bf16] panel
constexpr uint32_t kTileB = 2 * kPanelB;
constexpr int kBwdThreads = 384;
constexpr float kLog2eB = 1.4426950408889634f;

struct BwdSmem {
    alignas(1024) uint8_t x[kTileB];
    alignas(1024) uint8_t y[kTileB];
    alignas(1024) uint8_t u[kRing][kTileB];
    alignas(1024) uint8_t w[kRing][kTileB];
    alignas(16) float lse2[kRing][kTile];      // WHICH >= 1: per streamed query column
    alignas(16) float delta[kRing][kTile];
    alignas(8) uint64_t xy_full;
    uint64_t uw_full[kRing], uw_empty[kRing];
    uint64_t s_full, ld_done, p_full, acc_done;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

struct BwdParams {
    uint16_t* out0;        // dQ (WHICH 0) or dK (WHICH 1): contiguous [B, S, H, D]
    uint16_t* out1;        // dV (WHICH 1, 2)
    float* dq_accum;       // single-pass form: fp32 [B, Hq, S, D], zeroed before the launch
    const float* lse2;     // workspace plane 0: [B, Hq, S rounded up to whole tiles]
    const float* delta;    // workspace plane 1
    int batch, seq, q_heads, kv_heads;
    int causal;
    int rows_fastest;      // grid = (row tiles, heads, batch) instead of (heads, row tiles, batch)
    int softcap_grad;      // 0 analytical derivative of the polynomial, 1 the identity 1 - t^2
    float scale, softcap;
    float score_to_log2;   // scale * log2(e): raw score -> log2-domain score (plain softmax)
    float score_to_tanh;   // scale / softcap: raw score -> tanh argument
    float tanh_to_log2;    // softcap * log2(e): tanh value -> log2-domain score
    float sigmoid_mul, sigmoid_add;   // native sigmoid: p = 1 / (1 + 2^(score * sigmoid_mul + sigmoid_add))
    uint32_t tanh_dw[4];   // derivative of the tanh program as packed bf16 words: d0 + d1 t + d2 t^2 + d3 t^3
    uint32_t* status;
    ProgramWords tanh;
    B3Words b3;
};

// Optional timeline for tuning builds (-DFPT_ATTN_TRACE): block (0,0,0) stores (tag, SM clock) pairs behind the status
// word, 4096 words per traced warp and kernel; the caller must then pass a status buffer of 128 KiB.
#ifdef FPT_ATTN_TRACE
#define FPT_BTRACE(slot, tag)                                                                             \
    do {                                                                                                  \
        if (trace_on && lane == 0 && trace_n < 2046) {                                                    \
            uint32_t* t_ = p.status + 64 + ((slot) + 3 * WHICH) * 4096;                                   \
            t_[2 + trace_n] = uint32_t(tag);                                                              \
            t_[3 + trace_n] = uint32_t(clock64());                                                        \
            trace_n += 2;                                                                                 \
            t_[0] = uint32_t(trace_n);                                                                    \
        }                                                                                                 \
    } while (0)
#else
#define FPT_BTRACE(slot, tag) do { } while (0)
#endif

enum : uint32_t { kBwdXY = 1, kBwdUwEmpty, kBwdUwFull, kBwdSFull, kBwdPFull, kBwdAccDone, kBwdLdDone };

// 16 bytes to shared memory (address from smem_u32)
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t a) {
    asm volatile("st.shared.b32 [%0], %1;" :: "r"(addr), "r"(a) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ float ex2f(float x) { return mufu_ex2(x); }

// ---- pre-pass: lse2 = lse * log2(e), delta = sum_d dO * O, one warp per (batch, head, row) ------------------
struct PrepassArgs {
    const uint16_t* out;
    const uint16_t* dout;
    const float* lse;       // [B, Hq, S]
    float* lse2;
    float* delta;
    int64_t o_stride_b, o_stride_s, o_stride_h, do_stride_b, do_stride_s, do_stride_h;
    int batch, seq, seq_pad, q_heads;
};

__global__ void __launch_bounds__(256) attention_bwd_prepass_kernel(const PrepassArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = int64_t(a.batch) * a.q_heads * a.seq_pad;   // planes are padded to whole tiles
#pragma unroll 1
    for (int64_t row = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += int64_t(gridDim.x) * 8) {
        const int s = int(row % a.seq_pad);
        const int64_t bh = row / a.seq_pad;
        if (s >= a.seq) {                      // padding rows: defined values, so that nothing downstream meets a NaN
            if (lane == 0) {
                a.delta[row] = 0.0f;
                a.lse2[row] = 0.0f;
            }
            continue;
        }
        const int h = int(bh % a.q_heads), b = int(bh / a.q_heads);
        const uint2 o = *reinterpret_cast<const uint2*>(a.out + b * a.o_stride_b + s * a.o_stride_s + h * a.o_stride_h + lane * 4);
        const uint2 d = *reinterpret_cast<const uint2*>(a.dout + b * a.do_stride_b + s * a.do_stride_s + h * a.do_stride_h + lane * 4);
        float acc = Sfu<kBf16>::lo(o.x) * Sfu<kBf16>::lo(d.x);
        acc = fmaf(Sfu<kBf16>::hi(o.x), Sfu<kBf16>::hi(d.x), acc);
        acc = fmaf(Sfu<kBf16>::lo(o.y), Sfu<kBf16>::lo(d.y), acc);
        acc = fmaf(Sfu<kBf16>::hi(o.y), Sfu<kBf16>::hi(d.y), acc);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) {
            a.delta[row] = acc;
            a.lse2[row] = a.lse[bh * a.seq + s] * kLog2eB;
        }
    }
}

// ---- last pass of the fused form: dq [B, S, Hq, 128] = bf16(scale * accumulated fp32 dQ [B, Hq, S, 128]), eight elements
// per thread and step ----------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attention_bwd_dq_convert_kernel(const float* __restrict__ accum, uint16_t* __restrict__ dq,
                                                                      int64_t n8, int seq, int heads, float scale) {
#pragma unroll 1
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < n8; i += int64_t(gridDim.x) * 256) {
        const int d8 = int(i % (kDim / 8));
        const int64_t row = i / (kDim / 8);                 // (b, s, h) of the output
        const int h = int(row % heads);
        const int64_t bs = row / heads;
        const int sq = int(bs % seq);
        const int64_t b = bs / seq;
        const float4* src = reinterpret_cast<const float4*>(accum + ((b * heads + h) * seq + sq) * kDim) + 2 * d8;
        const float4 a = src[0], c = src[1];
        uint4 o;
        o.x = Sfu<kBf16>::pack(a.x * scale, a.y * scale);
        o.y = Sfu<kBf16>::pack(a.z * scale, a.w * scale);
        o.z = Sfu<kBf16>::pack(c.x * scale, c.y * scale);
        o.w = Sfu<kBf16>::pack(c.z * scale, c.w * scale);
        reinterpret_cast<uint4*>(dq)[i] = o;
    }
}

// four consecutive floats from shared memory (address from smem_u32, 16-byte aligned)
__device__ __forceinline__ void lds128(uint32_t addr, float (&v)[4]) {
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(addr));
}

// bf16x2 of two fp32 values (low lane first)
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return Sfu<kBf16>::pack(lo, hi); }

// One pair of columns of one row: raw scores s0, s1 and dP values d0, d1 -> bf16x2 words of P and of dS (the factor
// `scale` common to every dS is applied once, in the epilogue).
//   l0, l1: lse * log2(e) of the two (row, column) positions' query;  t0, t1: their delta;  m0, m1: masked out
//   routed: this pair takes the software exponential EK instead of the special-function unit (plain soft-max only)
template <int MODE, int GRAD, int EK>
__device__ __forceinline__ void score_pair(const BwdParams& p, float s0, float s1, float d0, float d1, float l0, float l1,
                                           float t0, float t1, bool m0, bool m1, bool routed, uint32_t& p_word,
                                           uint32_t& ds_word) {
    // fp32 steps run two lanes per instruction (mul2 / sub2 / fma2): these loops are bound by issue slots
    if constexpr (MODE == 1) {
        float x0, x1;
        mul2(s0, s1, p.scale, p.scale, x0, x1);
        uint32_t grad;
        // infinite scores are made finite by the conversion (see b3_direct_with_grad_select_late)
        uint32_t pr = b3_direct_with_grad_select_late(Sfu<kBf16>::pack_satfinite(x0, x1), p.b3, grad);
        float g0, g1;
        unpack_bf16x2(grad, g0, g1);
        mul2(g0, g1, d0, d1, g0, g1);
        if (m0) { pr &= 0xffff0000u; g0 = 0.0f; }
        if (m1) { pr &= 0x0000ffffu; g1 = 0.0f; }
        p_word = pr;
        ds_word = pack_bf16(g0, g1);
    } else if constexpr (MODE == 4) {
        // native twin of the direct cubic: p = sigmoid(score*scale - ln n) through ex2 and rcp, dS = dP p (1 - p)
        float a0, a1;
        fma2(s0, s1, p.sigmoid_mul, p.sigmoid_mul, p.sigmoid_add, p.sigmoid_add, a0, a1);
        float p0 = mufu_rcp(1.0f + ex2f(a0)), p1 = mufu_rcp(1.0f + ex2f(a1));
        if (m0) p0 = 0.0f;
        if (m1) p1 = 0.0f;
        float g0, g1;
        fma2(-p0, -p1, p0, p1, p0, p1, g0, g1);          // p - p^2
        mul2(g0, g1, d0, d1, g0, g1);
        p_word = pack_bf16(p0, p1);
        ds_word = pack_bf16(g0, g1);
    } else if constexpr (MODE == 2) {
        const float c = p.score_to_log2;
        float a0, a1, e0, e1;
        fma2(s0, s1, c, c, -l0, -l1, a0, a1);
        float p0, p1;
        if (routed) {
            exp2_full_x2<EK>(a0, a1, p0, p1);
        } else {
            p0 = ex2f(a0);
            p1 = ex2f(a1);
        }
        if (m0) p0 = 0.0f;
        if (m1) p1 = 0.0f;
        p_word = pack_bf16(p0, p1);
        sub2(d0, d1, t0, t1, e0, e1);
        mul2(p0, p1, e0, e1, e0, e1);
        ds_word = pack_bf16(e0, e1);
    } else {
        const float in = p.score_to_tanh, out = p.tanh_to_log2;
        float x0, x1;
        mul2(s0, s1, in, in, x0, x1);
        if constexpr (MODE == 3) {
            // native twin: tanh on the special-function unit, derivative 1 - t^2 of its value
            const float th0 = mufu_tanh(x0), th1 = mufu_tanh(x1);
            float a0, a1, g0, g1, e0, e1;
            fma2(th0, th1, out, out, -l0, -l1, a0, a1);
            float p0 = ex2f(a0), p1 = ex2f(a1);
            if (m0) p0 = 0.0f;
            if (m1) p1 = 0.0f;
            fma2(-th0, -th1, th0, th1, 1.0f, 1.0f, g0, g1);
            p_word = pack_bf16(p0, p1);
            sub2(d0, d1, t0, t1, e0, e1);
            mul2(p0, p1, e0, e1, e0, e1);
            mul2(e0, e1, g0, g1, e0, e1);
            ds_word = pack_bf16(e0, e1);
            return;
        }
        const uint32_t x = pack_bf16(x0, x1);
        // The saturating odd program written out (the same operations in the same order as eval_program<kBf16, kOddSat,
        // 4>), because its clamped argument c and its unsigned result also feed the derivative below.
        using P = Pk<kBf16>;
        const uint32_t c = P::min_abs(x, p.tanh.clamp);
        uint32_t h = P::fma(c, p.tanh.c[3], p.tanh.c[2]);
        h = P::fma(c, h, p.tanh.c[1]);
        h = P::fma(c, h, p.tanh.c[0]);
        const uint32_t sat = P::min(P::mul(c, h), Consts<kBf16>::one);
        const uint32_t th = sat ^ (x & kSignMask);
        float th0, th1, a0, a1;
        unpack_bf16x2(th, th0, th1);
        fma2(th0, th1, out, out, -l0, -l1, a0, a1);
        float p0 = ex2f(a0), p1 = ex2f(a1);
        if (m0) p0 = 0.0f;
        if (m1) p1 = 0.0f;
        p_word = pack_bf16(p0, p1);
        float e0, e1;
        sub2(d0, d1, t0, t1, e0, e1);
        mul2(p0, p1, e0, e1, e0, e1);
        if constexpr (GRAD == 1) {
            float g0, g1;
            fma2(-th0, -th1, th0, th1, 1.0f, 1.0f, g0, g1);
            mul2(e0, e1, g0, g1, e0, e1);
            ds_word = pack_bf16(e0, e1);
        } else {
            // derivative of the polynomial on packed bf16 lanes, like the polynomial itself: three fused
            // multiply-adds per pair; zero where the input is clamped or the output saturated (flat regions).  It
            // multiplies the packed P (dP - delta) directly (one packed multiply instead of unpacking the derivative and
            // multiplying in fp32: the product is rounded to bf16 either way, its first factor once more)
            uint32_t gw = P::fma(c, p.tanh_dw[3], p.tanh_dw[2]);
            gw = P::fma(c, gw, p.tanh_dw[1]);
            gw = P::fma(c, gw, p.tanh_dw[0]);
            gw &= ~(P::ge_mask(c, p.tanh.clamp) | P::ge_mask(sat, Consts<kBf16>::one));
            ds_word = P::mul(pack_bf16(e0, e1), gw);
        }
    }
}

// Tensor-memory columns.  WHICH 0 (dQ): S 0..127, two dP tiles 128..255 and 256..383, acc0 384..511.  WHICH 1 (dK, dV):
// S 0..127, one dP tile 128..255, acc0 (dK) 256..383, acc1 (dV) 384..511.  Inside a dP tile each column half (64 fp32
// columns = the 64 keys or queries of one score-mod warp per lane quarter) is overwritten by that warp's own results:
// 32 columns of bf16 dS pairs, then 32 columns of bf16 P pairs; the products read K steps 0..3 from the first half and
// 4..7 from the second.
constexpr uint32_t kColS = 0, kColDp = 128, kColAcc1 = 384;
template <int WHICH>
struct Cols {
    static constexpr uint32_t acc0 = WHICH == 0 ? 384u : 256u;
    static __device__ __forceinline__ uint32_t dp(int t) { return WHICH == 0 ? kColDp + 128u * uint32_t(t & 1) : kColDp; }
};

// GRAD (soft-capped mode only): 0 the analytical derivative of the tanh polynomial, 1 the identity 1 - t^2; a template
// parameter because the choice sits inside the per-pair arithmetic.
// EMU, EK (plain soft-max only): routing frequency and kind of the software exponential, as in the forward: four of
// every EMU columns of a score-mod warp's 64 take exp2_full_x2<EK> on the FMA pipe (reference: exp2_emu_freq_bwd,
// src/sfu_repro/fa4.py:724-752).
template <int MODE, int WHICH, int GRAD = 0, int EMU = 0, int EK = kExp2FullD3>
__global__ void __launch_bounds__(kBwdThreads, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                     const __grid_constant__ CUtensorMap map_u, const __grid_constant__ CUtensorMap map_w,
                     const BwdParams p) {
    constexpr bool kSigmoidMode = MODE == 1 || MODE == 4;    // no normalisation: neither lse nor delta
    constexpr bool kKeysFixed = WHICH == 1;                   // rows of the fixed tiles are keys, streamed tiles are queries
    using Smem = BwdSmem;
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are handed out x fastest: with row tiles on x the blocks that run together stream the same head's tiles,
    // which then come from L2; with heads on x they share their loop length (causal).
    const int head = p.rows_fastest ? blockIdx.y : blockIdx.x;                  // query head (WHICH 0) or kv head (WHICH 1)
    const int n_row_tiles = p.rows_fastest ? gridDim.x : gridDim.y, tile_id = p.rows_fastest ? blockIdx.x : blockIdx.y;
    const int tile = p.causal && !kKeysFixed ? n_row_tiles - 1 - tile_id : tile_id;  // long loops first
    const int b = blockIdx.z;
    const int total = (p.seq + kTile - 1) / kTile;   // a ragged last tile is zero-filled by TMA and masked below
    const int seq_pad = total * kTile;
    const bool ragged = (p.seq % kTile) != 0;
    const int group = p.q_heads / p.kv_heads;
    const int row0 = tile * kTile;                // first row of the fixed tiles
    // inner loop: WHICH 0 walks key tiles 0..(causal ? tile : total-1); WHICH 1 walks, for each query head of the
    // group, query tiles (causal ? tile : 0)..total-1
    const int first_inner = (kKeysFixed && p.causal) ? tile : 0;
    const int per_head = !kKeysFixed ? (p.causal ? tile + 1 : total) : total - first_inner;
    const int n_inner = !kKeysFixed ? per_head : per_head * group;
    const int fixed_head_x = head;
    const int stream_head0 = !kKeysFixed ? head / group : head * group;
    volatile uint32_t* abort_flag = &sm.abort_flag;
#ifdef FPT_ATTN_TRACE
    const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (warp == 1 || warp == 4 || warp == 8);
    int trace_n = 0;
#endif

    if (threadIdx.x == 0) {
        mbar_init(&sm.xy_full, 1);
        for (int st = 0; st < kRing; ++st) {
            mbar_init(&sm.uw_full[st], 1);
            mbar_init(&sm.uw_empty[st], 1);
        }
        mbar_init(&sm.s_full, 1);
        mbar_init(&sm.ld_done, 8);      // one arrive per score-mod warp: its S and dP values are in registers
        mbar_init(&sm.p_full, 8);       // one arrive per score-mod warp: its P and dS words are in tensor memory
        mbar_init(&sm.acc_done, 1);
        sm.abort_flag = *reinterpret_cast<volatile uint32_t*>(p.status) != 0u ? 1u : 0u;
        mbar_fence_init();
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_y);
        tma_prefetch_descriptor(&map_u);
        tma_prefetch_descriptor(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(&sm.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const bool skip = sm.abort_flag != 0u;

    // Register budget (see the forward kernel): 384 threads start at 168 and move 128 x (168 - 80) to the score-mod warps
    // (208 each).
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
      if (skip || warp >= 2) {
        // warps 2 and 3 only hold registers for the others
      } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(&sm.xy_full, 2 * kTileB);
            tma_load_4d(sm.x, &map_x, &sm.xy_full, 0, row0, fixed_head_x, b);
            tma_load_4d(sm.x + kPanelB, &map_x, &sm.xy_full, 64, row0, fixed_head_x, b);
            tma_load_4d(sm.y, &map_y, &sm.xy_full, 0, row0, fixed_head_x, b);
            tma_load_4d(sm.y + kPanelB, &map_y, &sm.xy_full, 64, row0, fixed_head_x, b);
            bool ok = true;
            for (int t = 0; t < n_inner && ok; ++t) {
                const int st = t % kRing;
                const uint32_t ph = uint32_t(t / kRing) & 1u;
                if (t >= kRing) ok = mbar_wait(&sm.uw_empty[st], ph ^ 1u, abort_flag, p.status, kBwdUwEmpty);
                if (!ok) break;
                const int g = !kKeysFixed ? 0 : t / per_head;
                const int r0 = (first_inner + (!kKeysFixed ? t : t - g * per_head)) * kTile;
                const int sh = stream_head0 + g;
                const uint32_t vec_bytes = kKeysFixed && !kSigmoidMode ? 2u * kTile * 4u : 0u;
                mbar_arrive_expect_tx(&sm.uw_full[st], 2 * kTileB + vec_bytes);
                tma_load_4d(sm.u[st], &map_u, &sm.uw_full[st], 0, r0, sh, b);
                tma_load_4d(sm.u[st] + kPanelB, &map_u, &sm.uw_full[st], 64, r0, sh, b);
                if (vec_bytes) {   // per-query vectors of the streamed query tile
                    const int64_t off = (int64_t(b) * p.q_heads + sh) * seq_pad + r0;
                    bulk_load_1d(sm.lse2[st], p.lse2 + off, kTile * 4u, &sm.uw_full[st]);
                    bulk_load_1d(sm.delta[st], p.delta + off, kTile * 4u, &sm.uw_full[st]);
                }
                tma_load_4d(sm.w[st], &map_w, &sm.uw_full[st], 0, r0, sh, b);
                tma_load_4d(sm.w[st] + kPanelB, &map_w, &sm.uw_full[st], 64, r0, sh, b);
            }
        }
      } else {
        // ------------------------------------------------------------------ UMMA issuer
        // The whole warp runs the loop (waits included) and one elected lane issues: see elect_one().
        {
            const bool elected = elect_one();
            constexpr uint32_t idesc_kk = umma_idesc_bf16(kTile, kTile, 0, 0);   // both operands K-major
            constexpr uint32_t idesc_mn = umma_idesc_bf16(kTile, kDim, 0, 1);    // B operand MN-major
            constexpr uint32_t desc_hi = umma_smem_desc_hi(1024);
            constexpr uint32_t kColAcc0 = Cols<WHICH>::acc0;
            auto dp_col = [](int t) { return Cols<WHICH>::dp(t); };
            const uint32_t x_lo = umma_smem_desc_lo(smem_u32(sm.x), 16), y_lo = umma_smem_desc_lo(smem_u32(sm.y), 16);
            // Software pipeline.  S is not aliased by anything (P sits in the upper half of the dP tile, WHICH 1, or
            // is not stored at all, WHICH 0), so S of step t+1 is issued as soon as the score-mod warps have S of
            // step t in registers.  WHICH 0 also has room for two dP tiles and issues dP of step t+1 at the same
            // point; WHICH 1 issues it behind the products that read dS and P of step t from that tile.
            auto stage_words = [&](int st, uint32_t& u_k, uint32_t& w_k, uint32_t& u_mn, uint32_t& w_mn) {
                u_k = umma_smem_desc_lo(smem_u32(sm.u[st]), 16);
                w_k = umma_smem_desc_lo(smem_u32(sm.w[st]), 16);
                u_mn = umma_smem_desc_lo(smem_u32(sm.u[st]), kPanelB);
                w_mn = umma_smem_desc_lo(smem_u32(sm.w[st]), kPanelB);
            };
            auto issue_s = [&](uint32_t u_k) {           // S = X U^T
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (uint32_t(kk >> 2) * kPanelB + uint32_t(kk & 3) * 32u) / 16u;
                    if (elected) umma_ss_words(tmem + kColS, x_lo + off, u_k + off, desc_hi, idesc_kk, kk > 0);
                }
            };
            auto issue_dp = [&](uint32_t w_k, int t) {   // dP = Y W^T into the tile of step t
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (uint32_t(kk >> 2) * kPanelB + uint32_t(kk & 3) * 32u) / 16u;
                    if (elected) umma_ss_words(tmem + dp_col(t), y_lo + off, w_k + off, desc_hi, idesc_kk, kk > 0);
                }
            };
            bool ok = mbar_wait(&sm.xy_full, 0, abort_flag, p.status, kBwdXY);
            uint32_t u_k = 0, w_k = 0, u_mn = 0, w_mn = 0;
            if (ok) ok = mbar_wait(&sm.uw_full[0], 0, abort_flag, p.status, kBwdUwFull);
            if (ok) {
                tc_fence_after_sync();
                stage_words(0, u_k, w_k, u_mn, w_mn);
                issue_s(u_k);
                issue_dp(w_k, 0);
                if (elected) umma_commit(&sm.s_full);
            }
            for (int t = 0; t < n_inner && ok; ++t) {
                const int st = t % kRing, st_next = (t + 1) % kRing;
                const bool more = t + 1 < n_inner;
                uint32_t nu_k = 0, nw_k = 0, nu_mn = 0, nw_mn = 0;
                // [A] S (and dP) of step t are in registers: S of step t+1 may overwrite S
                ok = mbar_wait(&sm.ld_done, uint32_t(t) & 1u, abort_flag, p.status, kBwdLdDone);
                if (!ok) break;
                FPT_BTRACE(2, 10);
                if (more) {
                    ok = mbar_wait(&sm.uw_full[st_next], uint32_t((t + 1) / kRing) & 1u, abort_flag, p.status, kBwdUwFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    stage_words(st_next, nu_k, nw_k, nu_mn, nw_mn);
                    issue_s(nu_k);
                    if constexpr (WHICH == 0) {
                        issue_dp(nw_k, t + 1);
                        if (elected) umma_commit(&sm.s_full);
                    }
                }
                FPT_BTRACE(2, 11);
                // [B] dS (and P) of step t are in tensor memory
                ok = mbar_wait(&sm.p_full, uint32_t(t) & 1u, abort_flag, p.status, kBwdPFull);
                if (!ok) break;
                tc_fence_after_sync();
                FPT_BTRACE(2, 12);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)       // acc0 += dS U
                    if (elected) umma_ts_words(tmem + kColAcc0, tmem + dp_col(t) + 64u * (kk >> 2) + 8u * (kk & 3),
                                  u_mn + uint32_t(kk) * (2048u / 16u), desc_hi, idesc_mn, t > 0 || kk > 0);
                if constexpr (kKeysFixed) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)   // acc1 += P W
                        if (elected) umma_ts_words(tmem + kColAcc1, tmem + dp_col(t) + 64u * (kk >> 2) + 32u + 8u * (kk & 3),
                                      w_mn + uint32_t(kk) * (2048u / 16u), desc_hi, idesc_mn, t > 0 || kk > 0);
                }
                if (elected) umma_commit(&sm.uw_empty[st]);
                FPT_BTRACE(2, 13);
                // [C] WHICH 1: the one dP tile is free again once the products above have read it (same thread, in order)
                if constexpr (kKeysFixed) {
                    if (more) {
                        issue_dp(nw_k, t + 1);
                        if (elected) umma_commit(&sm.s_full);
                    }
                }
                u_k = nu_k; w_k = nw_k; u_mn = nu_mn; w_mn = nw_mn;
            }
            if (ok && elected) umma_commit(&sm.acc_done);
        }
      }
    } else {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
      if (!skip) {
        // ------------------------------------------------------------------ score-mod warps
        const int quarter = warp & 3, half = (warp - 4) >> 2;
        const int r = 32 * quarter + lane;                       // row of the fixed tile = tensor-memory lane
        const uint32_t lane_base = uint32_t(32 * quarter) << 16;
        const uint32_t t_s = tmem + lane_base + kColS + uint32_t(64 * half);
        float row_lse2 = 0.0f, row_delta = 0.0f;
        if (!kKeysFixed && !kSigmoidMode) {
            const int64_t off = (int64_t(b) * p.q_heads + head) * seq_pad + row0 + r;
            row_lse2 = p.lse2[off];
            row_delta = p.delta[off];
        }
        bool ok = true;
        for (int t = 0; t < n_inner && ok; ++t) {
            const int st = t % kRing;
            FPT_BTRACE(half, 1);
            ok = mbar_wait(&sm.s_full, uint32_t(t) & 1u, abort_flag, p.status, kBwdSFull);
            if (!ok) break;
            tc_fence_after_sync();
            FPT_BTRACE(half, 2);
            // This warp owns columns [64 half, 64 half + 64) of the dP tile: it reads its dP values from there and writes
            // its bf16 dS words over the first 32 and its bf16 P words over the last 32 of them, so no other warp's loads
            // are in the way and nobody waits for anybody.  S and dP are read in full first; then the issuer is told
            // at once (S of the next step can start under this step's arithmetic), and the results leave in two chunks.
            uint32_t dv[64], sv[64];
            const uint32_t t_own = tmem + lane_base + Cols<WHICH>::dp(t) + uint32_t(64 * half);
            tmem_ld_32x32b_x32(t_own, reinterpret_cast<uint32_t(&)[32]>(dv[0]));
            tmem_ld_32x32b_x32(t_own + 32, reinterpret_cast<uint32_t(&)[32]>(dv[32]));
            tmem_ld_32x32b_x32(t_s, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
            tmem_ld_32x32b_x32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sv[32]));
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.ld_done);
            FPT_BTRACE(half, 3);
            if (kKeysFixed && !kSigmoidMode)   // the per-query vectors arrived on this barrier (already complete here)
                ok = mbar_wait(&sm.uw_full[st], uint32_t(t / kRing) & 1u, abort_flag, p.status, kBwdUwFull);
            if (!ok) break;
            const int g = !kKeysFixed ? 0 : t / per_head;
            const int c0 = (first_inner + (!kKeysFixed ? t : t - g * per_head)) * kTile + 64 * half;   // first column
            // tiles that need a mask: the causal diagonal, and any tile pair that touches a ragged end of the sequence
            const int tile_c0 = c0 - 64 * half;
            const bool diagonal = (p.causal && tile_c0 == row0) ||
                                  (ragged && (tile_c0 + kTile > p.seq || row0 + kTile > p.seq));
            const uint32_t lse_addr = smem_u32(&sm.lse2[st][64 * half]), delta_addr = smem_u32(&sm.delta[st][64 * half]);
            // results leave in two chunks of 16 words where the arithmetic is light (plain softmax: the stores overlap the
            // second chunk's exponentials) and in one piece where it is heavy (measured: the instruction-bound modes lose
            // about 10 % when their arithmetic is cut in two by the stores)
            constexpr bool kChunkedStores = MODE == 2 && EMU == 0;
            uint32_t pw[32], dsw[32];
#pragma unroll
            for (int chunk = 0; chunk < 2; ++chunk) {
                auto columns = [&](auto masked) {
#pragma unroll
                    for (int quad = 0; quad < 8; ++quad) {       // four columns = two pairs per 128-bit shared load
                        const int cq = 32 * chunk + 4 * quad;
                        float lv[4] = {row_lse2, row_lse2, row_lse2, row_lse2};
                        float dl[4] = {row_delta, row_delta, row_delta, row_delta};
                        if (kKeysFixed && !kSigmoidMode) {
                            lds128(lse_addr + 4u * cq, lv);
                            lds128(delta_addr + 4u * cq, dl);
                        }
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2) {
                            const int c = cq + 2 * h2;           // column pair inside this half
                            bool m0 = false, m1 = false;
                            if constexpr (decltype(masked)::value) {   // rows are queries (WHICH 0) or keys (WHICH 1)
                                const int row_abs = row0 + r, col_abs = c0 + c;
                                const int query0 = !kKeysFixed ? row_abs : col_abs, key0 = !kKeysFixed ? col_abs : row_abs;
                                const int query1 = !kKeysFixed ? row_abs : col_abs + 1, key1 = !kKeysFixed ? col_abs + 1 : row_abs;
                                m0 = (p.causal && key0 > query0) || key0 >= p.seq || query0 >= p.seq;
                                m1 = (p.causal && key1 > query1) || key1 >= p.seq || query1 >= p.seq;
                            }
                            const bool routed = EMU > 0 && ((c / 2) % (EMU > 0 ? EMU / 2 : 1)) < 2;
                            score_pair<MODE, GRAD, EK>(p, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), __uint_as_float(dv[c]),
                                             __uint_as_float(dv[c + 1]), lv[2 * h2], lv[2 * h2 + 1], dl[2 * h2], dl[2 * h2 + 1],
                                             m0, m1, routed, pw[16 * chunk + 2 * quad + h2], dsw[16 * chunk + 2 * quad + h2]);
                        }
                    }
                };
                if (diagonal) columns(std::true_type{});    // a branch the whole CTA takes together
                else columns(std::false_type{});
                if constexpr (kChunkedStores) {
                    tmem_st_32x32b_x16(t_own + 16 * chunk, reinterpret_cast<const uint32_t(&)[16]>(dsw[16 * chunk]));
                    if constexpr (kKeysFixed)                  // only dK / dV need P itself
                        tmem_st_32x32b_x16(t_own + 32 + 16 * chunk, reinterpret_cast<const uint32_t(&)[16]>(pw[16 * chunk]));
                }
            }
            if constexpr (!kChunkedStores) {
                tmem_st_32x32b_x32(t_own, dsw);
                if constexpr (kKeysFixed) tmem_st_32x32b_x32(t_own + 32, pw);
            }
            FPT_BTRACE(half, 5);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_full);
            FPT_BTRACE(half, 6);
        }
        if (ok && n_inner > 0) {
            ok = mbar_wait(&sm.acc_done, 0, abort_flag, p.status, kBwdAccDone);
            if (ok) {
                tc_fence_after_sync();
                const int64_t heads_out = !kKeysFixed ? p.q_heads : p.kv_heads;
                const int64_t off = ((int64_t(b) * p.seq + row0 + r) * heads_out + head) * kDim + 64 * half;
                const bool real_row = row0 + r < p.seq;
#pragma unroll
                for (int acc = 0; acc <= (kKeysFixed ? 1 : 0); ++acc) {
                    const float f = acc == 0 ? p.scale : 1.0f;
                    uint16_t* dst = (acc == 0 ? p.out0 : p.out1) + off;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(tmem + lane_base + (acc == 0 ? Cols<WHICH>::acc0 : kColAcc1) + uint32_t(64 * half + 32 * c), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 o;
                            o.x = pack_bf16(__uint_as_float(v[q4 * 8 + 0]) * f, __uint_as_float(v[q4 * 8 + 1]) * f);
                            o.y = pack_bf16(__uint_as_float(v[q4 * 8 + 2]) * f, __uint_as_float(v[q4 * 8 + 3]) * f);
                            o.z = pack_bf16(__uint_as_float(v[q4 * 8 + 4]) * f, __uint_as_float(v[q4 * 8 + 5]) * f);
                            o.w = pack_bf16(__uint_as_float(v[q4 * 8 + 6]) * f, __uint_as_float(v[q4 * 8 + 7]) * f);
                            if (real_row) reinterpret_cast<uint4*>(dst + 32 * c)[q4] = o;
                        }
                    }
                }
            }
        }
      }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}


// ---- single pass, pipelined by half steps ---------------------------------------------------------------------------------
// dK, dV and dQ in one kernel (5 matrix products per tile pair), one CTA per (batch, kv head, 128 keys), looping over the
// query heads of the group and their query tiles like WHICH = 1.  A step (one streamed 128-query tile) is cut into two
// half steps of 64 queries; S^T and dP^T of a half step take 64 tensor-memory columns each and there are two buffers of
// each (S 0..127, dP 128..255, dK 256..383, dV 384..511), so the tensor core computes the three products of half step n and
// then S^T and dP^T of half step n + 2 while the score-mod warps work on half step n + 1: the serial chain of a form with
// one S and one dP tile (dP product -> score-mod -> products -> dP of the next step) is gone and a step costs what the
// slower of the two sides costs, not their sum.  dQ^T of a half step is written over its S buffer (in registers since the
// start of its score-mod pass), so the dP buffer is free for half step n + 2 as soon as the products that read dS and P
// from it have been issued, and the wait for the read-out of dQ^T falls under the dP^T product.  (An M = 128, N = 64 product
// takes 49-54 cycles where an N = 128 one takes 64: the price of the two buffers.)
//   S^T_n  = K Q_n^T, dP^T_n = V dO_n^T                      (M = 128 keys, N = 64 queries, both operands K-major)
//   dK += dS^T_n Q_n, dV += P^T_n dO_n                        (A from tensor memory, B MN-major; 4 K steps of 16 queries)
//   dQ^T_n = K^T dS^T_n                                       (M = 128 head-dim, N = 64 queries, both operands MN-major; into
//                                                              the S buffer of the half step)
// Roles: warp 0 TMA producer, warp 1 issuer (converged, an elected lane issues), warps 4..11 score-mod (thread = key row;
// warps w and w + 4 split the 64 queries of a half step), warps 12..19 read-out of dQ^T (lane = head-dim index) in two
// warpgroups, one per 32 queries of a half step: registers (the columns are released at once), then the team's 16 KiB
// staging buffer (512 bytes per query, the layout of the head-major fp32 buffer) and one untiled reduce-add copy, which
// the team waits for only when it needs the buffer again.  (One warpgroup doing both chunks of a half step took ~3000
// cycles per half step on schedulers it shares with the score-mod warps and held the whole pipeline to that.)  The streamed
// Q / dO ring holds half tiles (64 queries), three stages.  The dS^T tile in shared memory is one panel ([keys x 64
// queries]) reused by every half step: it is written at the end of a score-mod pass, long after the dQ^T product of the
// half step before has read it.
constexpr int kPipeRing = 3;       // half-tile stages of the streamed Q / dO ring
constexpr int kPipeStaging = 2;    // staging buffers of the read-out: one per read-out warpgroup
constexpr uint32_t kHalfPanelB = kPanelB / 2;   // one [64 rows x 64 bf16] panel

struct PipeSmem {
    alignas(1024) uint8_t x[kTileB];            // K tile
    alignas(1024) uint8_t y[kTileB];            // V tile
    alignas(1024) uint8_t u[kPipeRing][kPanelB];    // Q half tiles (64 queries): two panels of [64 rows x 64 bf16]
    alignas(1024) uint8_t w[kPipeRing][kPanelB];    // dO half tiles
    alignas(1024) uint8_t ds[kPanelB];              // dS^T of one half step, bf16, swizzled
    alignas(1024) uint8_t stage[kPipeStaging][kPanelB];   // 32 queries x 128 fp32 of a partial dQ tile on their way out
    alignas(16) float lse2[kPipeRing][kTile / 2];
    alignas(16) float delta[kPipeRing][kTile / 2];
    alignas(8) uint64_t xy_full;
    uint64_t uw_full[kPipeRing], uw_empty[kPipeRing];
    uint64_t sd_full[2];      // S^T and dP^T of a half step are complete (per buffer)
    uint64_t p_full[2];       // 8 warps: dS and P words in tensor memory, dS^T in shared memory
    uint64_t dq_full[2];      // dQ^T of a half step complete (and with it everything that read the dS^T tile)
    uint64_t dq_read[2];      // 4 warps: dQ^T in registers (the S buffer it was written over is free)
    uint64_t staged[kPipeStaging];       // 4 warps: 32 queries are in the staging buffer
    uint64_t stage_free[kPipeStaging];   // the copy engine has read them
    uint64_t acc_done;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

enum : uint32_t { kPipeSdFull = 16, kPipePFull, kPipeDqFull, kPipeDqRead, kPipeStaged, kPipeStageFree };

// SMW: score-mod warps, 8 (two per lane quarter, 32 queries of a half step each) or 16 (four per lane quarter, 16 queries each)
constexpr int pipe_threads(int smw) { return 128 + 32 * smw + 256; }

template <int MODE, int GRAD = 0, int EMU = 0, int EK = kExp2FullD3, int SMW = 8>
__global__ void __launch_bounds__(pipe_threads(SMW), 1)
attention_bwd_pipelined_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                               const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                               const BwdParams p) {
    constexpr bool kSigmoidMode = MODE == 1 || MODE == 4;
    constexpr int kHalf = kTile / 2;                      // queries of a half step
    static_assert(SMW == 8 || SMW == 16, "two or four score-mod warps per lane quarter");
    constexpr int kCols = kHalf / (SMW / 4);              // queries of a half step per score-mod warp: 32 or 16
    constexpr int kFirstReadOut = 4 + SMW;                // first read-out warp
    extern __shared__ uint8_t smem_raw[];
    // the shared memory of an SM is filled to the last kilobyte: no alignment slack, the base is checked below
    PipeSmem& sm = *reinterpret_cast<PipeSmem*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = p.rows_fastest ? blockIdx.y : blockIdx.x;                  // kv head
    const int tile = p.rows_fastest ? blockIdx.x : blockIdx.y;                  // key tile
    const int b = blockIdx.z;
    const int total = (p.seq + kTile - 1) / kTile;
    const int seq_pad = total * kTile;
    const bool ragged = (p.seq % kTile) != 0;
    const int group = p.q_heads / p.kv_heads;
    const int row0 = tile * kTile;                        // first key
    const int first_inner = p.causal ? tile : 0;          // first query tile
    const int per_head = total - first_inner;
    const int n_inner = per_head * group;
    const int n_half = 2 * n_inner;
    const int stream_head0 = head * group;
    volatile uint32_t* abort_flag = &sm.abort_flag;
#ifdef FPT_ATTN_TRACE
    constexpr int WHICH = 2;      // trace slots 6..9
    const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (warp == 1 || warp == 4 || warp == 8 || warp == kFirstReadOut);
    int trace_n = 0;
#endif

    if (threadIdx.x == 0) {
        mbar_init(&sm.xy_full, 1);
        for (int st = 0; st < kPipeRing; ++st) {
            mbar_init(&sm.uw_full[st], 1);
            mbar_init(&sm.uw_empty[st], 1);
        }
        for (int i = 0; i < kPipeStaging; ++i) {
            mbar_init(&sm.staged[i], 4);
            mbar_init(&sm.stage_free[i], 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(&sm.sd_full[h], 1);
            mbar_init(&sm.p_full[h], SMW);
            mbar_init(&sm.dq_full[h], 1);
            mbar_init(&sm.dq_read[h], 8);
        }
        mbar_init(&sm.acc_done, 1);
        sm.abort_flag = *reinterpret_cast<volatile uint32_t*>(p.status) != 0u ? 1u : 0u;
        if ((smem_u32(&sm) & 1023u) != 0u) {              // the operand layouts need 1024-byte alignment
            sm.abort_flag = 1u;
            atomicCAS(p.status, 0u, 0x80000000u | kBwdXY | 0x100u);
        }
        mbar_fence_init();
        tma_prefetch_descriptor(&map_k);
        tma_prefetch_descriptor(&map_v);
        tma_prefetch_descriptor(&map_q);
        tma_prefetch_descriptor(&map_do);
    }
    if (warp == 1) {
        tmem_alloc(&sm.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const bool skip = sm.abort_flag != 0u;
    constexpr uint32_t kS = 0, kDp = 128, kAcc0 = 256, kAcc1 = 384;   // tensor-memory columns

    // 640 (896) threads start at 96 (72) registers each.  The producer / issuer warpgroup and the two read-out warpgroups give
    // registers back, the score-mod warpgroups take them; an increase waits until the registers are there, so the sums must
    // work out.
    constexpr int kThreadsAll = pipe_threads(SMW);
    constexpr int kRegsStart = SMW == 8 ? 96 : 72, kRegsWg0 = SMW == 8 ? 56 : 48, kRegsReadOut = SMW == 8 ? 80 : 64;
    constexpr int kRegsScoreMod = SMW == 8 ? 128 : 80;
    static_assert(65536 / kThreadsAll / 8 * 8 == kRegsStart, "registers per thread at launch");
    static_assert(128 * (kRegsStart - kRegsWg0) + 256 * (kRegsStart - kRegsReadOut) >= 32 * SMW * (kRegsScoreMod - kRegsStart),
                  "register hand-over: more taken than released would block the score-mod warps for ever");
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kRegsWg0));
      if (skip || warp >= 2) {
        // warps 2 and 3 only hold registers for the others
      } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(&sm.xy_full, 2 * kTileB);
            tma_load_4d(sm.x, &map_k, &sm.xy_full, 0, row0, head, b);
            tma_load_4d(sm.x + kPanelB, &map_k, &sm.xy_full, 64, row0, head, b);
            tma_load_4d(sm.y, &map_v, &sm.xy_full, 0, row0, head, b);
            tma_load_4d(sm.y + kPanelB, &map_v, &sm.xy_full, 64, row0, head, b);
            bool ok = true;
            for (int n = 0; n < n_half && ok; ++n) {      // one ring stage per half step: 64 queries of Q and of dO
                const int t = n >> 1, h = n & 1, st = n % kPipeRing;
                const uint32_t ph = uint32_t(n / kPipeRing) & 1u;
                if (n >= kPipeRing) ok = mbar_wait(&sm.uw_empty[st], ph ^ 1u, abort_flag, p.status, kBwdUwEmpty);
                if (!ok) break;
                const int g = t / per_head;
                const int r0 = (first_inner + (t - g * per_head)) * kTile + kHalf * h;   // may lie past the end: zero fill
                const int sh = stream_head0 + g;
                const uint32_t vec_bytes = !kSigmoidMode ? 2u * kHalf * 4u : 0u;
                mbar_arrive_expect_tx(&sm.uw_full[st], kTileB + vec_bytes);
                tma_load_4d(sm.u[st], &map_q, &sm.uw_full[st], 0, r0, sh, b);
                tma_load_4d(sm.u[st] + kHalfPanelB, &map_q, &sm.uw_full[st], 64, r0, sh, b);
                tma_load_4d(sm.w[st], &map_do, &sm.uw_full[st], 0, r0, sh, b);
                tma_load_4d(sm.w[st] + kHalfPanelB, &map_do, &sm.uw_full[st], 64, r0, sh, b);
                if (vec_bytes) {   // per-query vectors of the 64 queries (the planes are padded to whole tiles)
                    const int64_t off = (int64_t(b) * p.q_heads + sh) * seq_pad + r0;
                    bulk_load_1d(sm.lse2[st], p.lse2 + off, kHalf * 4u, &sm.uw_full[st]);
                    bulk_load_1d(sm.delta[st], p.delta + off, kHalf * 4u, &sm.uw_full[st]);
                }
            }
        }
      } else {
        // ------------------------------------------------------------------ UMMA issuer
        // The whole warp runs the loop (waits included) and one elected lane issues: see elect_one().
        {
            const bool elected = elect_one();
            constexpr uint32_t idesc_kk = umma_idesc_bf16(kTile, kHalf, 0, 0);     // S^T, dP^T: both operands K-major
            constexpr uint32_t idesc_mn = umma_idesc_bf16(kTile, kDim, 0, 1);      // dK, dV: B operand MN-major
            constexpr uint32_t idesc_mnmn = umma_idesc_bf16(kDim, kHalf, 1, 1);    // dQ^T: both operands MN-major
            constexpr uint32_t desc_hi = umma_smem_desc_hi(1024);
            const uint32_t x_k = umma_smem_desc_lo(smem_u32(sm.x), 16), y_k = umma_smem_desc_lo(smem_u32(sm.y), 16);
            const uint32_t x_mn = umma_smem_desc_lo(smem_u32(sm.x), kPanelB);
            const uint32_t ds_mn = umma_smem_desc_lo(smem_u32(sm.ds), kPanelB);
            // K step k of a half step (16 queries) belongs to score-mod warp k / (kCols / 16) of each lane quarter, which keeps
            // its dS words in the first half of its own kCols dP columns and its P words in the second half
            auto a_col = [](int k) { return uint32_t(kCols * (k / (kCols / 16)) + 8 * (k % (kCols / 16))); };
            // K-major operand, K step kk of 16 head-dim elements: panel kk / 4 (16 KiB apart in the fixed tiles, 8 KiB in the
            // half tiles of the ring), 32 bytes per step inside the 128-byte line
            auto issue_s = [&](int st, int h) {
                const uint32_t u_k = umma_smem_desc_lo(smem_u32(sm.u[st]), 16);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t in = uint32_t(kk & 3) * 32u;
                    if (elected) umma_ss_words(tmem + kS + uint32_t(kHalf * h), x_k + (uint32_t(kk >> 2) * kPanelB + in) / 16u,
                                  u_k + (uint32_t(kk >> 2) * kHalfPanelB + in) / 16u, desc_hi, idesc_kk, kk > 0);
                }
            };
            auto issue_dp = [&](int st, int h) {
                const uint32_t w_k = umma_smem_desc_lo(smem_u32(sm.w[st]), 16);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t in = uint32_t(kk & 3) * 32u;
                    if (elected) umma_ss_words(tmem + kDp + uint32_t(kHalf * h), y_k + (uint32_t(kk >> 2) * kPanelB + in) / 16u,
                                  w_k + (uint32_t(kk >> 2) * kHalfPanelB + in) / 16u, desc_hi, idesc_kk, kk > 0);
                }
            };
            bool ok = mbar_wait(&sm.xy_full, 0, abort_flag, p.status, kBwdXY);
            // S^T and dP^T of the first two half steps (both buffers are free)
            for (int n = 0; n < 2 && n < n_half && ok; ++n) {
                ok = mbar_wait(&sm.uw_full[n], 0, abort_flag, p.status, kBwdUwFull);
                if (!ok) break;
                tc_fence_after_sync();
                issue_s(n, n);
                issue_dp(n, n);
                if (elected) umma_commit(&sm.sd_full[n]);
            }
            for (int n = 0; n < n_half && ok; ++n) {
                const int t = n >> 1, h = n & 1, st = n % kPipeRing;
                FPT_BTRACE(2, 10);
                // dS, P (tensor memory) and dS^T (shared memory) of this half step are written
                ok = mbar_wait(&sm.p_full[h], uint32_t(t) & 1u, abort_flag, p.status, kPipePFull);
                if (!ok) break;
                tc_fence_after_sync();
                FPT_BTRACE(2, 15);
                const uint32_t u_mn = umma_smem_desc_lo(smem_u32(sm.u[st]), kHalfPanelB);
                const uint32_t w_mn = umma_smem_desc_lo(smem_u32(sm.w[st]), kHalfPanelB);
                const uint32_t a_base = tmem + kDp + uint32_t(kHalf * h);
#pragma unroll
                for (int k = 0; k < 4; ++k)          // dK += dS^T Q: 16 queries per K step, out of the columns of the warp that wrote them
                    if (elected) umma_ts_words(tmem + kAcc0, a_base + a_col(k), u_mn + uint32_t(k) * (2048u / 16u),
                                  desc_hi, idesc_mn, n > 0 || k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k)          // dV += P^T dO
                    if (elected) umma_ts_words(tmem + kAcc1, a_base + a_col(k) + uint32_t(kCols / 2), w_mn + uint32_t(k) * (2048u / 16u),
                                  desc_hi, idesc_mn, n > 0 || k > 0);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)       // dQ^T = K^T dS^T over the S buffer of the half step (in registers long ago)
                    if (elected) umma_ss_words(tmem + kS + uint32_t(kHalf * h), x_mn + uint32_t(kk) * (2048u / 16u),
                                  ds_mn + uint32_t(kk) * (2048u / 16u), desc_hi, idesc_mnmn, kk > 0);
                if (elected) umma_commit(&sm.dq_full[h]);
                FPT_BTRACE(2, 16);
                if (elected) umma_commit(&sm.uw_empty[st]);       // every product that reads the stage is behind this commit
                if (n + 2 < n_half) {
                    // S^T and dP^T of the half step after the next one, into this half step's buffers.  The dP buffer is free
                    // as soon as the two products above have read dS and P from it (issued before, executed in order); the S
                    // buffer once the read-out warps have taken dQ^T out of it, which happens under the dP^T product.
                    const int n2 = n + 2, st2 = n2 % kPipeRing;
                    ok = mbar_wait(&sm.uw_full[st2], uint32_t(n2 / kPipeRing) & 1u, abort_flag, p.status, kBwdUwFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    FPT_BTRACE(2, 11);
                    issue_dp(st2, h);
                    FPT_BTRACE(2, 12);
                    ok = mbar_wait(&sm.dq_read[h], uint32_t(t) & 1u, abort_flag, p.status, kPipeDqRead);
                    if (!ok) break;
                    tc_fence_after_sync();
                    FPT_BTRACE(2, 13);
                    issue_s(st2, h);
                    if (elected) umma_commit(&sm.sd_full[h]);
                    FPT_BTRACE(2, 14);
                }
            }
            if (ok && elected) umma_commit(&sm.acc_done);
        }
      }
    } else if (warp >= kFirstReadOut) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kRegsReadOut));
      if (!skip) {
        // ------------------------------------------------------------------ read-out warps
        // Two warpgroups: team 0 (the first four warps) takes queries 0..31 of every half step, team 1 queries 32..63,
        // each through its own 16 KiB staging buffer and its own reduce-add copy per half step.  The tensor-memory columns
        // are released as soon as both teams have their values in registers; the copy of a half step is waited for (by the
        // team's issuing lane) only when the buffer is needed again, after the next release.
        const int team = (warp - kFirstReadOut) >> 2, quarter = warp & 3;
        const bool issuing = quarter == 0;                  // the team's first warp hands the staged chunk to the copy engine
        const uint32_t lane_base = uint32_t(32 * quarter) << 16;
        const uint32_t mine = smem_u32(sm.stage[team]) + uint32_t(32 * quarter + lane) * 4u;
        bool ok = true;
        for (int n = 0; n < n_half && ok; ++n) {
            const int t = n >> 1, h = n & 1;
            const int g = t / per_head;
            const int q0 = (first_inner + (t - g * per_head)) * kTile + kHalf * h + 32 * team;     // first query of the chunk
            ok = mbar_wait(&sm.dq_full[h], uint32_t(t) & 1u, abort_flag, p.status, kPipeDqFull);
            if (!ok) break;
            tc_fence_after_sync();
            FPT_BTRACE(3, 20);
            uint32_t v[32];
            tmem_ld_32x32b_x32(tmem + lane_base + kS + uint32_t(kHalf * h + 32 * team), v);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.dq_read[h]);
            FPT_BTRACE(3, 21);
            if (n > 0) {                                    // the copy of the half step before has read the buffer
                if (issuing && lane == 0) {
                    bulk_wait_group_read0();
                    mbar_arrive(&sm.stage_free[team]);
                }
                ok = mbar_wait(&sm.stage_free[team], uint32_t(n - 1) & 1u, abort_flag, p.status, kPipeStageFree);
                if (!ok) break;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) sts32(mine + uint32_t(j) * (kDim * 4u), v[j]);
            fence_async_shared();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.staged[team]);
            if (issuing) {
                if (lane == 0) {
                    ok = mbar_wait(&sm.staged[team], uint32_t(n) & 1u, abort_flag, p.status, kPipeStaged);
                    const int rows = min(32, p.seq - q0);
                    float* dst = p.dq_accum + ((int64_t(b) * p.q_heads + stream_head0 + g) * p.seq + q0) * kDim;
#ifndef FPT_DIAG_NO_RED
                    if (ok && rows > 0) bulk_reduce_add_f32_1d(dst, sm.stage[team], uint32_t(rows) * (kDim * 4u));
#endif
                    bulk_commit_group();
                }
                ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
                FPT_BTRACE(3, 22);
            }
        }
        if (issuing && lane == 0) bulk_wait_group0();
      }
    } else {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" :: "n"(kRegsScoreMod));
      if (!skip) {
        // ------------------------------------------------------------------ score-mod warps
        const int quarter = warp & 3, cw = (warp - 4) >> 2;          // lane quarter; which kCols of a half step's 64 queries
        const int r = 32 * quarter + lane;                           // key row of the tile = tensor-memory lane
        const uint32_t lane_base = uint32_t(32 * quarter) << 16;
        bool ok = true;
        for (int n = 0; n < n_half && ok; ++n) {
            const int t = n >> 1, h = n & 1, st = n % kPipeRing;
            ok = mbar_wait(&sm.sd_full[h], uint32_t(t) & 1u, abort_flag, p.status, kPipeSdFull);
            if (!ok) break;
            tc_fence_after_sync();
            FPT_BTRACE(cw & 1, 2);
            // This warp owns columns [kCols cw, kCols cw + kCols) of the half step's S and dP buffers; it writes its dS words
            // over the first half and its P words over the second half of its own dP columns, so nobody's loads are in the way.
            uint32_t dv[kCols], sv[kCols];
            const uint32_t t_own = tmem + lane_base + kDp + uint32_t(kHalf * h + kCols * cw);
            const uint32_t t_s = tmem + lane_base + kS + uint32_t(kHalf * h + kCols * cw);
            if constexpr (kCols == 32) {
                tmem_ld_32x32b_x32(t_own, dv);
                tmem_ld_32x32b_x32(t_s, sv);
            } else {
                tmem_ld_32x32b_x16(t_own, dv);
                tmem_ld_32x32b_x16(t_s, sv);
            }
            tmem_ld_wait();
            FPT_BTRACE(cw & 1, 3);
            if (!kSigmoidMode)                 // the per-query vectors arrived on this barrier (complete by now)
                ok = mbar_wait(&sm.uw_full[st], uint32_t(n / kPipeRing) & 1u, abort_flag, p.status, kBwdUwFull);
            if (!ok) break;
            const int g = t / per_head;
            const int tile_c0 = (first_inner + (t - g * per_head)) * kTile;        // first query of the streamed tile
            const int in_tile = kHalf * h + kCols * cw;                            // this warp's first query inside it
            const int c0 = tile_c0 + in_tile;
            const bool diagonal = (p.causal && tile_c0 == row0) || (ragged && (tile_c0 + kTile > p.seq || row0 + kTile > p.seq));
            const uint32_t lse_addr = smem_u32(&sm.lse2[st][kCols * cw]), delta_addr = smem_u32(&sm.delta[st][kCols * cw]);
            uint32_t pw[kCols / 2], dsw[kCols / 2];
            auto columns = [&](auto masked) {
#pragma unroll
                for (int quad = 0; quad < kCols / 4; ++quad) {       // four queries = two pairs per 128-bit shared load
                    const int cq = 4 * quad;
                    float lv[4] = {0.0f, 0.0f, 0.0f, 0.0f}, dl[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (!kSigmoidMode) {
                        lds128(lse_addr + 4u * cq, lv);
                        lds128(delta_addr + 4u * cq, dl);
                    }
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int c = cq + 2 * h2;
                        bool m0 = false, m1 = false;
                        if constexpr (decltype(masked)::value) {
                            const int key = row0 + r, query0 = c0 + c, query1 = c0 + c + 1;
                            m0 = (p.causal && key > query0) || key >= p.seq || query0 >= p.seq;
                            m1 = (p.causal && key > query1) || key >= p.seq || query1 >= p.seq;
                        }
                        const bool routed = EMU > 0 && ((c / 2) % (EMU > 0 ? EMU / 2 : 1)) < 2;
                        score_pair<MODE, GRAD, EK>(p, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), __uint_as_float(dv[c]),
                                                   __uint_as_float(dv[c + 1]), lv[2 * h2], lv[2 * h2 + 1], dl[2 * h2], dl[2 * h2 + 1],
                                                   m0, m1, routed, pw[2 * quad + h2], dsw[2 * quad + h2]);
                    }
                }
            };
            if (diagonal) columns(std::true_type{});    // a branch the whole CTA takes together
            else columns(std::false_type{});
            FPT_BTRACE(cw & 1, 4);
            if constexpr (kCols == 32) {
                tmem_st_32x32b_x16(t_own, dsw);
                tmem_st_32x32b_x16(t_own + 16, pw);
            } else {
                tmem_st_32x32b_x8(t_own, dsw);
                tmem_st_32x32b_x8(t_own + 8, pw);
            }
            // dS^T also goes to shared memory for the dQ^T product: this thread's key row, its kCols queries = kCols / 8
            // chunks of the row's 128-byte line, chunk j stored at position j ^ (row % 8) (the 128-byte swizzle of the
            // operand layout).  The tile is free once the dQ^T product of the half step before is complete.
            if (n > 0) ok = mbar_wait(&sm.dq_full[h ^ 1], uint32_t((n - 1) >> 1) & 1u, abort_flag, p.status, kPipeDqFull);
            if (!ok) break;
            FPT_BTRACE(cw & 1, 5);
            const uint32_t line = smem_u32(sm.ds) + uint32_t(r) * 128u;
#pragma unroll
            for (int j = 0; j < kCols / 8; ++j)
                sts128(line + (uint32_t(((kCols / 8) * cw + j) ^ (r & 7)) << 4), dsw[4 * j], dsw[4 * j + 1], dsw[4 * j + 2],
                       dsw[4 * j + 3]);
            fence_async_shared();
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_full[h]);
            FPT_BTRACE(cw & 1, 6);
        }
        if (ok && n_half > 0) {
            ok = mbar_wait(&sm.acc_done, 0, abort_flag, p.status, kBwdAccDone);
            if (ok) {
                tc_fence_after_sync();
                constexpr int kOutCols = kDim / (SMW / 4);      // head-dimension columns of dK and dV this warp writes out
                const int64_t off = ((int64_t(b) * p.seq + row0 + r) * p.kv_heads + head) * kDim + kOutCols * cw;
                const bool real_row = row0 + r < p.seq;
#pragma unroll
                for (int acc = 0; acc < 2; ++acc) {
                    const float f = acc == 0 ? p.scale : 1.0f;
                    uint16_t* dst = (acc == 0 ? p.out0 : p.out1) + off;
#pragma unroll
                    for (int c = 0; c < kOutCols / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(tmem + lane_base + (acc == 0 ? kAcc0 : kAcc1) + uint32_t(kOutCols * cw + 32 * c), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 o;
                            o.x = pack_bf16(__uint_as_float(v[q4 * 8 + 0]) * f, __uint_as_float(v[q4 * 8 + 1]) * f);
                            o.y = pack_bf16(__uint_as_float(v[q4 * 8 + 2]) * f, __uint_as_float(v[q4 * 8 + 3]) * f);
                            o.z = pack_bf16(__uint_as_float(v[q4 * 8 + 4]) * f, __uint_as_float(v[q4 * 8 + 5]) * f);
                            o.w = pack_bf16(__uint_as_float(v[q4 * 8 + 6]) * f, __uint_as_float(v[q4 * 8 + 7]) * f);
                            if (real_row) reinterpret_cast<uint4*>(dst + 32 * c)[q4] = o;
                        }
                    }
                }
            }
        }
      }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace fpt

using namespace fpt;

// two planes [B, Hq, S padded to whole tiles] fp32 (lse * log2 e, delta)
static int64_t bwd_planes_bytes(int64_t batch, int64_t seq, int64_t q_heads) {
    const int64_t seq_pad = (seq + kTile - 1) / kTile * kTile;
    return 2 * batch * q_heads * seq_pad * int64_t(sizeof(float));
}

extern "C" int64_t fpt_attention_bwd_workspace_bytes(int64_t batch, int64_t seq, int64_t q_heads) {
    if (batch <= 0 || seq <= 0 || q_heads <= 0) return 0;
    return bwd_planes_bytes(batch, seq, q_heads);
}

// the planes, then the fp32 dQ buffer [B, S, Hq, 128] of the single-pass form
extern "C" int64_t fpt_attention_bwd_fused_workspace_bytes(int64_t batch, int64_t seq, int64_t q_heads) {
    if (batch <= 0 || seq <= 0 || q_heads <= 0) return 0;
    return bwd_planes_bytes(batch, seq, q_heads) + batch * seq * q_heads * kDim * int64_t(sizeof(float));
}

extern "C" int fpt_attention_bwd_routed(void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k,
                                        const void* v, const void* out, const void* lse, void* workspace,
                                        int64_t workspace_bytes, int64_t batch, int64_t seq, int64_t q_heads,
                                        int64_t kv_heads, int64_t head_dim, const int64_t* q_strides,
                                        const int64_t* k_strides, const int64_t* v_strides, const int64_t* out_strides,
                                        const int64_t* dout_strides, int mode, int causal, float scale, float softcap,
                                        int log2_n, int softcap_grad, int exp2_emu_backend, int exp2_emu_freq,
                                        void* status, fpt_stream_t stream) {
    if (!dq || !dk || !dv || !dout || !q || !k || !v || !status || !q_strides || !k_strides || !v_strides || !dout_strides)
        return FPT_ERR_NULL_POINTER;
    if (batch <= 0 || seq <= 0 || q_heads <= 0 || kv_heads <= 0) return FPT_ERR_BAD_SIZE;
    if (head_dim != kDim || q_heads % kv_heads != 0) return FPT_ERR_UNSUPPORTED_SHAPE;
    if (batch > 65535 || q_heads > 0x7fffffff || seq > 0x3fffffff) return FPT_ERR_BAD_SIZE;
    if (mode < FPT_ATTN_SOFTCAP_TANH || mode > FPT_ATTN_SIGMOID_NATIVE) return FPT_ERR_BAD_ENUM;
    const bool softcap_family = mode == FPT_ATTN_SOFTCAP_TANH || mode == FPT_ATTN_SOFTCAP_NATIVE;
    const bool normalised = mode != FPT_ATTN_SIGMOID_DIRECT && mode != FPT_ATTN_SIGMOID_NATIVE;
    if (softcap_family && !(softcap > 0.0f)) return FPT_ERR_BAD_SIZE;
    if (!normalised && (log2_n < 1 || log2_n > 24)) return FPT_ERR_BAD_SIZE;
    if (softcap_grad != FPT_SOFTCAP_GRAD_ANALYTICAL && softcap_grad != FPT_SOFTCAP_GRAD_ONE_MINUS_T2) return FPT_ERR_BAD_ENUM;
    if (exp2_emu_freq != 0 && exp2_emu_freq != 8 && exp2_emu_freq != 12 && exp2_emu_freq != 16 && exp2_emu_freq != 32)
        return FPT_ERR_BAD_ENUM;
    if (exp2_emu_backend < FPT_EXP2_FULL_D3 || exp2_emu_backend > FPT_EXP2_FULL_PWL2_SAFE_F16) return FPT_ERR_BAD_ENUM;
    if (exp2_emu_freq != 0 && mode != FPT_ATTN_SOFTMAX) return FPT_ERR_BAD_ENUM;     // routed for the plain soft-max only
    if (normalised) {
        if (!out || !lse || !out_strides || !workspace) return FPT_ERR_NULL_POINTER;
        if (workspace_bytes < fpt_attention_bwd_workspace_bytes(batch, seq, q_heads)) return FPT_ERR_SCRATCH_TOO_SMALL;
        for (int i = 0; i < 3; ++i)
            if ((out_strides[i] * 2) & 7 || (dout_strides[i] * 2) & 7) return FPT_ERR_MISALIGNED;
        if ((reinterpret_cast<uintptr_t>(out) & 7u) || (reinterpret_cast<uintptr_t>(dout) & 7u)) return FPT_ERR_MISALIGNED;
    }
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15u)) return FPT_ERR_MISALIGNED;
    if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15u)
        return FPT_ERR_MISALIGNED;
    // the single-pass form (5 matrix products) runs when the caller's workspace also holds the fp32 dQ buffer and the
    // tuning key allows it; otherwise the two-pass form (7 products, deterministic), which needs the planes only
    const bool fused = workspace && workspace_bytes >= fpt_attention_bwd_fused_workspace_bytes(batch, seq, q_heads) &&
                       fpt::tuning_attention_bwd_fused() != 0;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;

    auto make_map = [&](CUtensorMap* map, const void* base, const int64_t* st, int64_t heads, uint32_t box_rows = kTile) {
        const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(seq), uint64_t(heads), uint64_t(batch)};
        const uint64_t strides[3] = {uint64_t(st[1]) * 2, uint64_t(st[2]) * 2, uint64_t(st[0]) * 2};
        return make_tensor_map_bf16_4d(map, base, dims, strides, box_rows);
    };
    CUtensorMap map_q, map_k, map_v, map_do;
    if (int rc = make_map(&map_q, q, q_strides, q_heads)) return rc;
    if (int rc = make_map(&map_k, k, k_strides, kv_heads)) return rc;
    if (int rc = make_map(&map_v, v, v_strides, kv_heads)) return rc;
    if (int rc = make_map(&map_do, dout, dout_strides, q_heads)) return rc;
    CUtensorMap map_q_half = map_q, map_do_half = map_do;      // 64-row boxes: the pipelined single-pass form streams half tiles
    if (fused) {
        if (int rc = make_map(&map_q_half, q, q_strides, q_heads, kTile / 2)) return rc;
        if (int rc = make_map(&map_do_half, dout, dout_strides, q_heads, kTile / 2)) return rc;
    }

    float* lse2 = static_cast<float*>(workspace);
    const int64_t seq_pad = (seq + kTile - 1) / kTile * kTile;
    float* delta = lse2 ? lse2 + batch * q_heads * seq_pad : nullptr;
    if (normalised) {
        PrepassArgs a{};
        a.out = static_cast<const uint16_t*>(out);
        a.dout = static_cast<const uint16_t*>(dout);
        a.lse = static_cast<const float*>(lse);
        a.lse2 = lse2;
        a.delta = delta;
        a.o_stride_b = out_strides[0]; a.o_stride_s = out_strides[1]; a.o_stride_h = out_strides[2];
        a.do_stride_b = dout_strides[0]; a.do_stride_s = dout_strides[1]; a.do_stride_h = dout_strides[2];
        a.batch = int(batch); a.seq = int(seq); a.seq_pad = int(seq_pad); a.q_heads = int(q_heads);
        int64_t grid = (batch * q_heads * seq_pad + 7) / 8;
        const int64_t cap = int64_t(dev.sm_count) * 32;
        if (grid > cap) grid = cap;
        attention_bwd_prepass_kernel<<<unsigned(grid), 256, 0, stream>>>(a);
        if (int rc = cuda_status(cudaGetLastError())) return rc;
    }

    BwdParams p{};
    p.lse2 = lse2;
    p.delta = delta;
    p.batch = int(batch); p.seq = int(seq); p.q_heads = int(q_heads); p.kv_heads = int(kv_heads);
    p.causal = causal ? 1 : 0;
    p.softcap_grad = softcap_grad;
    p.scale = scale; p.softcap = softcap;
    p.score_to_log2 = scale * kLog2eB;
    p.score_to_tanh = softcap != 0.0f ? scale / softcap : 0.0f;
    p.tanh_to_log2 = softcap * kLog2eB;
    p.status = static_cast<uint32_t*>(status);
    const ProgramRow* tanh_row = find_program(FPT_FN_TANH, FPT_FWD, 4, FPT_BF16, FPT_SRC_CURRENT);
    if (!tanh_row || tanh_row->shape != kOddSat) return FPT_ERR_UNKNOWN_PROGRAM;
    p.tanh = program_words(*tanh_row);
    // y = t (c1 + t (c2 + t (c3 + t c4)))  ->  dy/dt = c1 + 2 c2 t + 3 c3 t^2 + 4 c4 t^3, each coefficient rounded to
    // bf16 (nearest even) from the exact multiple of the program's bf16 coefficient
    auto scaled_bf16 = [](uint16_t bits, float factor) {
        uint32_t u = uint32_t(bits) << 16;
        float f;
        memcpy(&f, &u, 4);
        f *= factor;                                   // exact: a bf16 value times 1..4 fits in fp32
        memcpy(&u, &f, 4);
        u += 0x7fffu + ((u >> 16) & 1u);
        return (u >> 16) * 0x00010001u;
    };
    for (int i = 0; i < 4; ++i) p.tanh_dw[i] = scaled_bf16(tanh_row->c[i], float(i + 1));
    p.b3 = b3_words(mode == FPT_ATTN_SIGMOID_DIRECT ? log2_n : 12);
    p.sigmoid_mul = -scale * kLog2eB;
    p.sigmoid_add = float(log2_n);

    static_assert(sizeof(BwdSmem) + 1024 <= 227 * 1024, "shared memory budget");
    static_assert(sizeof(PipeSmem) <= 227 * 1024, "shared memory budget of the single-pass form (no alignment slack)");
    const unsigned tiles = unsigned(seq_pad / kTile);
    float* dq_accum = fused ? reinterpret_cast<float*>(static_cast<char*>(workspace) + bwd_planes_bytes(batch, seq, q_heads)) : nullptr;
    auto launch = [&](auto kernel, size_t smem, unsigned heads, const CUtensorMap& mx, const CUtensorMap& my,
                      const CUtensorMap& mu, const CUtensorMap& mw, uint16_t* o0, uint16_t* o1, unsigned threads = kBwdThreads) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
        BwdParams pp = p;
        pp.out0 = o0;
        pp.out1 = o1;
        pp.dq_accum = dq_accum;
        const dim3 grid = pp.rows_fastest ? dim3{tiles, heads, unsigned(batch)} : dim3{heads, tiles, unsigned(batch)};
        kernel<<<grid, threads, smem, stream>>>(mx, my, mu, mw, pp);
        return cuda_status(cudaGetLastError());
    };
    // Measured: with full (unmasked) attention over many heads, row tiles fastest is 10-12 % faster (B=2, S=16384, 32 heads:
    // the tiles one wave streams then belong to a few heads and stay in L2); with a causal mask heads fastest wins by 5-8 %
    // (blocks that run together have the same loop length), as it does while everything streamed fits L2 anyway.
    const int raster = fpt::tuning_attention_raster();
    const double streamed_all_heads = double(q_heads) * double(seq) * kDim * 2.0 * 2.0;
    p.rows_fastest = raster >= 0 ? raster : (!causal && streamed_all_heads > 64.0 * 1024 * 1024 ? 1 : 0);
    auto run = [&](auto mode_tag, auto grad_tag, auto emu_tag, auto kind_tag) {
        constexpr int M = decltype(mode_tag)::value;
        constexpr int G = decltype(grad_tag)::value;
        constexpr int E = decltype(emu_tag)::value;
        constexpr int EK = decltype(kind_tag)::value;
        if (fused) {
            // one pass: fixed K, V; streamed Q, dO; partial dQ tiles added into the fp32 buffer, then scaled and rounded
            const int64_t n = batch * seq * q_heads * kDim;
            cudaError_t e = cudaMemsetAsync(dq_accum, 0, size_t(n) * sizeof(float), stream);
            if (e != cudaSuccess) return int(e);
            // sixteen score-mod warps pay where the score-mod is heaviest (the polynomial soft-cap with its analytical
            // derivative: +7 % on the causal GQA workload) and cost 4-5 % elsewhere; tuning key value 2 forces them
            const bool wide = fpt::tuning_attention_bwd_fused() == 2 || (M == 0 && G == 0);
            const int rc = wide
                ? launch(attention_bwd_pipelined_kernel<M, G, E, EK, 16>, sizeof(PipeSmem), unsigned(kv_heads), map_k, map_v,
                         map_q_half, map_do_half, static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv), pipe_threads(16))
                : launch(attention_bwd_pipelined_kernel<M, G, E, EK, 8>, sizeof(PipeSmem), unsigned(kv_heads), map_k, map_v,
                         map_q_half, map_do_half, static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv), pipe_threads(8));
            if (rc) return rc;
            int64_t grid = (n / 8 + 255) / 256;
            const int64_t cap = int64_t(dev.sm_count) * 16;
            if (grid > cap) grid = cap;
            attention_bwd_dq_convert_kernel<<<unsigned(grid), 256, 0, stream>>>(dq_accum, static_cast<uint16_t*>(dq), n / 8, int(seq),
                                                                                int(q_heads), scale);
            return cuda_status(cudaGetLastError());
        }
        // dQ: fixed Q, dO; streamed K, V.   dK, dV: fixed K, V; streamed Q, dO
        const size_t smem = sizeof(BwdSmem) + 1024;
        if (int rc = launch(attention_bwd_kernel<M, 0, G, E, EK>, smem, unsigned(q_heads), map_q, map_do, map_k, map_v,
                            static_cast<uint16_t*>(dq), nullptr))
            return rc;
        return launch(attention_bwd_kernel<M, 1, G, E, EK>, smem, unsigned(kv_heads), map_k, map_v, map_q, map_do,
                      static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv));
    };
    if (mode == FPT_ATTN_SOFTCAP_TANH)
        return softcap_grad == 1 ? run(IC<0>{}, IC<1>{}, IC<0>{}, IC<0>{}) : run(IC<0>{}, IC<0>{}, IC<0>{}, IC<0>{});
    if (mode == FPT_ATTN_SIGMOID_DIRECT) return run(IC<1>{}, IC<0>{}, IC<0>{}, IC<0>{});
    if (mode == FPT_ATTN_SOFTCAP_NATIVE) return run(IC<3>{}, IC<0>{}, IC<0>{}, IC<0>{});
    if (mode == FPT_ATTN_SIGMOID_NATIVE) return run(IC<4>{}, IC<0>{}, IC<0>{}, IC<0>{});
    auto routed = [&](auto kind_tag) {
        switch (exp2_emu_freq) {
            case 8: return run(IC<2>{}, IC<0>{}, IC<8>{}, kind_tag);
            case 12: return run(IC<2>{}, IC<0>{}, IC<12>{}, kind_tag);
            case 16: return run(IC<2>{}, IC<0>{}, IC<16>{}, kind_tag);
            default: return run(IC<2>{}, IC<0>{}, IC<32>{}, kind_tag);
        }
    };
    if (exp2_emu_freq == 0) return run(IC<2>{}, IC<0>{}, IC<0>{}, IC<0>{});
    switch (exp2_emu_backend) {
        case FPT_EXP2_FULL_D3: return routed(IC<kExp2FullD3>{});
        case FPT_EXP2_FULL_PWL2: return routed(IC<kExp2FullPwl2>{});
        case FPT_EXP2_FULL_D2_SAFE: return routed(IC<kExp2FullD2Safe>{});
        default: return routed(IC<kExp2FullPwl2SafeF16>{});
    }
}

extern "C" int fpt_attention_bwd(void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k,
                                 const void* v, const void* out, const void* lse, void* workspace,
                                 int64_t workspace_bytes, int64_t batch, int64_t seq, int64_t q_heads, int64_t kv_heads,
                                 int64_t head_dim, const int64_t* q_strides, const int64_t* k_strides,
                                 const int64_t* v_strides, const int64_t* out_strides, const int64_t* dout_strides,
                                 int mode, int causal, float scale, float softcap, int log2_n, int softcap_grad,
                                 void* status, fpt_stream_t stream) {
    return fpt_attention_bwd_routed(dq, dk, dv, dout, q, k, v, out, lse, workspace, workspace_bytes, batch, seq, q_heads,
                                    kv_heads, head_dim, q_strides, k_strides, v_strides, out_strides, dout_strides, mode,
                                    causal, scale, softcap, log2_n, softcap_grad, FPT_EXP2_FULL_D3, 0, status, stream);
}
