// Attention forward for sm_100a with a polynomial score-mod on the softmax warps.
//
// One CTA owns 256 query rows (two 128-row tiles, "slots") of one (batch, query head) and walks the key/value
// sequence in tiles of 128 keys:
//   warp 0        TMA producer: Q once, then K and V tiles into a 2-stage shared-memory ring (no multicast)
//   warp 1        UMMA issuer (the warp runs converged, an elected lane issues): S = Q K^T into tensor memory,
//                 O += P V with P read from tensor memory
//   warps 2..3    idle (they complete the first warpgroup, which gives most of its registers away)
//   warps 4..7    softmax / score-mod warpgroup of slot 0 (thread = one query row = one tensor-memory lane)
//   warps 8..11   the same for slot 1
// Tensor memory (512 columns): S[slot] 128 fp32 columns each, O[slot] 128 fp32 columns each; the bf16 P tile of a
// slot overwrites the first 64 columns of its S tile once the row has been read into registers.  The two slots are
// interleaved on the tensor pipe so that one slot's matrix products run under the other slot's score-mod.
//
// Score-mods (all on packed bf16 lanes, FMA pipe):
//   mode 0  soft-capped softmax: s' = cap * tanh_D4(bf16(s*scale/cap)), then exp2 / running max / running sum
//   mode 1  sigmoid attention:   p = direct piecewise cubic of bf16(s*scale) (B3), no normalisation, O = P V
//   mode 2  plain softmax
// and their native twins on the special-function unit, the controls every polynomial number is compared with:
//   mode 3  soft-capped softmax with tanh.approx.f32 on the fp32 score (same layouts as mode 0)
//   mode 4  sigmoid attention with p = rcp(1 + ex2(log2 n - s*scale*log2 e)), two special-function operations per key
// Every mbarrier wait is bounded; on a timeout the CTA records where it stopped and unwinds.
#include <type_traits>

#include "fpt_common.h"
#include "fpt_programs.h"
#include "fpt_scoremod.cuh"
#include "fpt_sm100.cuh"

namespace fpt {
namespace {

using namespace sm100;

constexpr int kTileM = 128;          // query rows per slot
constexpr int kTileN = 128;          // keys per tile
constexpr int kHeadDim = 128;
constexpr int kSlots = 2;
constexpr int kStages = 2;
constexpr uint32_t kPanel = 128 * 128;        // bytes of one [128 rows x 64 bf16] panel
constexpr uint32_t kTileBytes = 2 * kPanel;   // one 128 x 128 bf16 tile
constexpr int kThreads = 128 * (1 + kSlots);  // warpgroup 0: producer + issuer; one warpgroup per slot
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;     // lazy rescale: tolerate exp2 arguments up to +8

struct AttnSmem {
    alignas(1024) uint8_t q[kSlots][kTileBytes];
    alignas(1024) uint8_t k[kStages][kTileBytes];
    alignas(1024) uint8_t v[kStages][kTileBytes];
    alignas(8) uint64_t q_full[kSlots];
    uint64_t k_full[2 * kStages], k_empty[2 * kStages], v_full[2 * kStages], v_empty[2 * kStages];   // a pair's half tiles: twice the stages
    uint64_t s_full[kSlots], p_half[kSlots], p_full[kSlots], pv_done[kSlots];
    uint64_t ld_done[kSlots];            // column-split variant: the eight warps of a slot have their S values in registers
    float xchg[kSlots][2][kTileM];       // column-split variant: row maximum / row sum of the other column half
    uint32_t tmem_base;
    uint32_t abort_flag;
};

struct AttnParams {
    uint16_t* out;       // (B, S, Hq, D) strides below, D contiguous
    float* lse;          // [B, Hq, S] or null
    int64_t out_stride_b, out_stride_s, out_stride_h;
    int batch, seq, q_heads, kv_heads;
    int mode, causal;
    int rows_fastest;    // grid = (row blocks, heads, batch) instead of (heads, row blocks, batch)
    float scale, softcap;
    float sigmoid_mul, sigmoid_add;   // native sigmoid: exponent = score * sigmoid_mul + sigmoid_add (log2 units)
    uint32_t* status;
    ProgramWords tanh;   // bf16 TANH_FWD_D4
    B3Words b3;
};

// EMU: routing frequency of the software exponential in the soft-max modes, with the meaning the reference gives
// exp2_emu_freq (reference: src/sfu_repro/fa4.py:724-733): 0 keeps every lane on the special-function unit; a positive
// frequency f sends four of every f keys of a row through a software exponential on the FMA pipe (12 -> one third,
// 32 -> one eighth); EK picks it: the cubic ("d3") or the two-piece line ("pwl2") of fpt_scoremod.cuh.  The unit
// delivers 16 results per clock and SM, which for a 128 x 128 tile takes as long as the two tensor-core products of
// that tile: that is the pressure the routing is meant to relieve.
// Optional timeline for tuning builds (-DFPT_ATTN_TRACE): block (0,0,0) stores (tag, SM clock) pairs behind the
// status word, 4096 words per traced warp; the caller must then pass a status buffer of 64 KiB.
#ifdef FPT_ATTN_TRACE
#define FPT_TRACE(slot, tag)                                                                              \
    do {                                                                                                  \
        if (trace_on && lane == 0 && trace_n < 2046) {                                                    \
            uint32_t* t_ = p.status + 64 + (slot) * 4096;                                                 \
            t_[2 + trace_n] = uint32_t(tag);                                                              \
            t_[3 + trace_n] = uint32_t(clock64());                                                        \
            trace_n += 2;                                                                                 \
            t_[0] = uint32_t(trace_n);                                                                    \
        }                                                                                                 \
    } while (0)
#else
#define FPT_TRACE(slot, tag) do { } while (0)
#endif

enum : uint32_t { kWhereQ = 1, kWhereKEmpty, kWhereVEmpty, kWhereKFull, kWhereVFull, kWherePFull, kWhereSFull, kWherePvDone };

__device__ __forceinline__ float ex2(float x) { return mufu_ex2(x); }

// mode families: the native twins share everything but the score-mod arithmetic with the polynomial modes
constexpr bool is_sigmoid(int mode) { return mode == 1 || mode == 4; }
constexpr bool is_softcap(int mode) { return mode == 0 || mode == 3; }

// native sigmoid of a pair of raw scores: two special-function operations per key (ex2, rcp)
__device__ __forceinline__ uint32_t native_sigmoid_pair(uint32_t s0, uint32_t s1, float mul, float add) {
    float a0, a1;
    asm("{\n\t.reg .b64 v, s, t, r;\n\t"
        "mov.b64 v, {%2, %3};\n\tmov.b64 s, {%4, %4};\n\tmov.b64 t, {%5, %5};\n\t"
        "fma.rn.f32x2 r, v, s, t;\n\tmov.b64 {%0, %1}, r;\n\t}"
        : "=f"(a0), "=f"(a1) : "r"(s0), "r"(s1), "f"(mul), "f"(add));
    const float p0 = mufu_rcp(1.0f + mufu_ex2(a0)), p1 = mufu_rcp(1.0f + mufu_ex2(a1));
    return Sfu<kBf16>::pack(p0, p1);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// bf16x2( a*scale, b*scale ) from two fp32 bit patterns: one packed fp32 multiply, one conversion
__device__ __forceinline__ uint32_t scale_pack_bf16x2(uint32_t a, uint32_t b, float scale) {
    uint32_t d;
    asm("{\n\t.reg .b64 v, s, r;\n\t.reg .b32 lo, hi;\n\t"
        "mov.b64 v, {%1, %2};\n\tmov.b64 s, {%3, %3};\n\t"
        "mul.rn.f32x2 r, v, s;\n\tmov.b64 {lo, hi}, r;\n\t"
        "cvt.rn.bf16x2.f32 %0, hi, lo;\n\t}"
        : "=r"(d) : "r"(a), "r"(b), "f"(scale));
    return d;
}
// (o0, o1) = (a0, a1) * m + c
__device__ __forceinline__ void fma_f32x2(float a0, float a1, float m, float c, float& o0, float& o1) {
    asm("{\n\t.reg .b64 v, s, t, r;\n\t"
        "mov.b64 v, {%2, %3};\n\tmov.b64 s, {%4, %4};\n\tmov.b64 t, {%5, %5};\n\t"
        "fma.rn.f32x2 r, v, s, t;\n\tmov.b64 {%0, %1}, r;\n\t}"
        : "=f"(o0), "=f"(o1) : "f"(a0), "f"(a1), "f"(m), "f"(c));
}
// (acc0, acc1) += (e0, e1)
__device__ __forceinline__ void add_f32x2(float& acc0, float& acc1, float e0, float e1) {
    asm("{\n\t.reg .b64 a, e;\n\t"
        "mov.b64 a, {%0, %1};\n\tmov.b64 e, {%2, %3};\n\t"
        "add.rn.f32x2 a, a, e;\n\tmov.b64 {%0, %1}, a;\n\t}"
        : "+f"(acc0), "+f"(acc1) : "f"(e0), "f"(e1));
}

// SPLIT: sixteen score-mod warps instead of eight; the two warps that share a lane quarter of a slot take 64 key
// columns each (keys 0..63 answer on the first hand-over barrier, keys 64..127 on the second).  It needs a mode without
// per-tile row reductions; the host uses it for the soft-capped mode with a bounded score range (fixed exponent
// reference, see below).
constexpr int kThreadsSplit = 128 + 256 * kSlots;
// soft-cap * log2(e) up to which the fixed reference cannot overflow or underflow (see the derivation at its use)
constexpr float kFixedReferenceLimit = 98.0f;
constexpr float kFixedReferenceSpan = 96.0f;

// PAIR: the block runs as one of a cluster of two (tcgen05 cta_group::2).  Both CTAs own 256 query rows as before (two
// heads of one K/V group, or two neighbouring row blocks of one head), and every product is ONE instruction of 256 rows
// issued by the first CTA: S = Q K^T reads each CTA's own Q and HALF of the key tile from each (keys 0..63 from the
// first CTA, 64..127 from the second), O += P V reads each CTA's own P and half of V's columns from each.  A CTA therefore
// loads and holds half of every K and V tile (map_kh: the K map with a 64-row box).  Loads of both CTAs complete on the
// first CTA's barriers, its commits reach both CTAs' barriers, and the score-mod warps of the second CTA announce their
// P tiles on the first CTA's barriers.  Same bits as the single-CTA kernel.  Measured 0.85-1.00x its speed at every shape
// (two or four ring stages, either wait scope): the kernel is not bound by the shared-memory reads this form halves, and
// a product that needs the P tiles of two CTAs waits for the slower of them.  Opt-in (tuning key "attention_cta_pair").
template <int MODE, int EMU, bool SPLIT, int EK = kExp2FullD3, bool PAIR = false>
__global__ void __launch_bounds__(SPLIT ? kThreadsSplit : kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_kh,
                     const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_cta_rank() : 0u;      // clusters of two along x
    // K / V ring: a CTA of a pair holds half of every tile, so the same shared memory gives it twice the stages
#ifndef FPT_ATTN_PAIR_STAGES
#define FPT_ATTN_PAIR_STAGES 4
#endif
    constexpr int kSt = PAIR ? FPT_ATTN_PAIR_STAGES : kStages;
    constexpr uint32_t kStageBytes = PAIR ? kTileBytes / 2 : kTileBytes;
    auto k_stage = [&](int st) { return &sm.k[0][0] + uint32_t(st) * kStageBytes; };
    auto v_stage = [&](int st) { return &sm.v[0][0] + uint32_t(st) * kStageBytes; };
    // Blocks are handed out x fastest.  With heads on x the blocks that run together share their length (causal) but walk
    // the K/V of every head at once; with row blocks on x they share one head's K/V, which then stays in L2.
    const int hq = p.rows_fastest ? blockIdx.y : blockIdx.x;
    const int n_qblocks = p.rows_fastest ? gridDim.x : gridDim.y;
    const int qb = p.rows_fastest ? blockIdx.x : blockIdx.y;
    const int qblock = p.causal ? n_qblocks - 1 - qb : qb;  // heavy causal blocks first
    const int b = blockIdx.z;
    const int hk = hq / (p.q_heads / p.kv_heads);
    const int m0 = qblock * (kSlots * kTileM);
    const int total_tiles = (p.seq + kTileN - 1) / kTileN;   // a ragged last tile is zero-filled by TMA and masked below
    int n_tiles[kSlots];
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
        const int row0 = m0 + s * kTileM;
        n_tiles[s] = row0 >= p.seq ? 0 : (p.causal ? min(total_tiles, row0 / kTileN + 1) : total_tiles);
    }
    const int n_max = max(n_tiles[0], n_tiles[1]);
    volatile uint32_t* abort_flag = &sm.abort_flag;
#ifdef FPT_ATTN_TRACE
    const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (warp == 1 || warp == 4 || warp == (SPLIT ? 12 : 8));
    int trace_n = 0;
#endif

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(&sm.q_full[s], 1);
            mbar_init(&sm.s_full[s], 1);
            mbar_init(&sm.p_half[s], PAIR ? 8 : 4);   // one arrive per softmax warp: keys 0..63 of the tile are in place
            mbar_init(&sm.p_full[s], PAIR ? 8 : 4);   // ... and keys 64..127 (PAIR: the warps of both CTAs)
            mbar_init(&sm.pv_done[s], 1);
            mbar_init(&sm.ld_done[s], 8);
        }
        for (int st = 0; st < kSt; ++st) {
            mbar_init(&sm.k_full[st], 1);
            mbar_init(&sm.k_empty[st], 1);
            mbar_init(&sm.v_full[st], 1);
            mbar_init(&sm.v_empty[st], 1);
        }
        // a CTA that starts after another one has reported a timeout does nothing, so that a fault in the
        // pipeline costs one wait limit and not one per CTA
        sm.abort_flag = *reinterpret_cast<volatile uint32_t*>(p.status) != 0u ? 1u : 0u;
        mbar_fence_init();
        tma_prefetch_descriptor(&map_q);
        tma_prefetch_descriptor(PAIR ? &map_kh : &map_k);
        tma_prefetch_descriptor(&map_v);
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tmem_alloc_pair(&sm.tmem_base, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(&sm.tmem_base, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    if constexpr (PAIR) cluster_sync_all();       // both CTAs' barriers exist before anything arrives from the other CTA
    else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const bool skip = sm.abort_flag != 0u;
    // "this warp's part of P is in tensor memory" (the warp has waited for its stores): to the issuing CTA's barrier; from the
    // second CTA of a pair without release semantics, which would wait for the K / V loads in flight into this CTA
    auto arrive_p = [&](uint64_t* bar) {
        if (!PAIR || rank == 0) mbar_arrive(bar);
        else mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(bar), 0));
    };

    // Register budget.  A CTA can only re-distribute the registers it was launched with (threads x the per-thread count
    // the launch bound allows): what the score-mod warps gain must have been given up by warpgroup 0 first, or
    // setmaxnreg.inc waits for ever.  384 threads: 168 at launch, 128 x (168-80) = 11264 released >= 256 x (208-168) = 10240
    // taken.  640 threads (column-split): 96 at launch, 128 x (96-56) = 5120 released >= 512 x (104-96) = 4096 taken.
    // Each setmaxnreg sits at the head of the branch it governs, so that the assembler knows which limit holds where.
    static_assert(128 * (168 - 80) >= 256 * (208 - 168) && 128 * (96 - 56) >= 512 * (104 - 96), "register hand-over");
    static_assert(65536 / kThreads / 8 * 8 == 168 && 65536 / kThreadsSplit / 8 * 8 == 96, "registers per thread at launch");
    if (warp < 4) {
      if constexpr (SPLIT) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
      else asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
      if (skip || warp >= 2) {
        // warps 2 and 3 only hold registers for the others; fall through to the teardown
      } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int s = 0; s < kSlots; ++s) {
                if (n_tiles[s] == 0) continue;
                if constexpr (PAIR) {
                    const uint32_t bar = map_to_cta(smem_u32(&sm.q_full[s]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&sm.q_full[s], 2 * kTileBytes);
                    tma_load_4d_pair(sm.q[s], &map_q, bar, 0, m0 + s * kTileM, hq, b);
                    tma_load_4d_pair(sm.q[s] + kPanel, &map_q, bar, 64, m0 + s * kTileM, hq, b);
                } else {
                    mbar_arrive_expect_tx(&sm.q_full[s], kTileBytes);
                    tma_load_4d(sm.q[s], &map_q, &sm.q_full[s], 0, m0 + s * kTileM, hq, b);
                    tma_load_4d(sm.q[s] + kPanel, &map_q, &sm.q_full[s], 64, m0 + s * kTileM, hq, b);
                }
            }
            bool ok = true;
            for (int j = 0; j < n_max && ok; ++j) {
                const int st = j % kSt;
                const uint32_t ph = uint32_t(j / kSt) & 1u;
                if (j >= kSt) ok = mbar_wait(&sm.k_empty[st], ph ^ 1u, abort_flag, p.status, kWhereKEmpty);
                if (!ok) break;
                if constexpr (PAIR) {      // this CTA's 64 keys of the tile: two panels [64 keys x 64 columns]
                    const uint32_t bar = map_to_cta(smem_u32(&sm.k_full[st]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&sm.k_full[st], kTileBytes);
                    tma_load_4d_pair(k_stage(st), &map_kh, bar, 0, j * kTileN + 64 * int(rank), hk, b);
                    tma_load_4d_pair(k_stage(st) + kPanel / 2, &map_kh, bar, 64, j * kTileN + 64 * int(rank), hk, b);
                } else {
                    mbar_arrive_expect_tx(&sm.k_full[st], kTileBytes);
                    tma_load_4d(sm.k[st], &map_k, &sm.k_full[st], 0, j * kTileN, hk, b);
                    tma_load_4d(sm.k[st] + kPanel, &map_k, &sm.k_full[st], 64, j * kTileN, hk, b);
                }
                if (j >= kSt) ok = mbar_wait(&sm.v_empty[st], ph ^ 1u, abort_flag, p.status, kWhereVEmpty);
                if (!ok) break;
                if constexpr (PAIR) {      // this CTA's 64 columns of V for all 128 keys: one panel
                    const uint32_t bar = map_to_cta(smem_u32(&sm.v_full[st]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&sm.v_full[st], kTileBytes);
                    tma_load_4d_pair(v_stage(st), &map_v, bar, 64 * int(rank), j * kTileN, hk, b);
                } else {
                    mbar_arrive_expect_tx(&sm.v_full[st], kTileBytes);
                    tma_load_4d(sm.v[st], &map_v, &sm.v_full[st], 0, j * kTileN, hk, b);
                    tma_load_4d(sm.v[st] + kPanel, &map_v, &sm.v_full[st], 64, j * kTileN, hk, b);
                }
            }
        }
      } else if (rank == 0) {
        // ------------------------------------------------------------------ UMMA issuer (PAIR: for both CTAs)
        // The whole warp runs the loop (waits included) and one elected lane issues: see elect_one().
        {
            const bool elected = elect_one();
            constexpr uint32_t idesc_qk = umma_idesc_bf16(PAIR ? 2 * kTileM : kTileM, kTileN, 0, 0);
            constexpr uint32_t idesc_pv = umma_idesc_bf16(PAIR ? 2 * kTileM : kTileM, kHeadDim, 0, 1);
            constexpr uint32_t k_panel = PAIR ? kPanel / 2 : kPanel;    // a CTA of a pair holds 64 keys of a tile
            auto commit = [&](uint64_t* bar) {
                if (elected) {
                    if constexpr (PAIR) umma_commit_pair(bar, 3);
                    else umma_commit(bar);
                }
            };
            // P tiles are announced by the warps of both CTAs of a pair
            auto wait_p = [&](uint64_t* bar, uint32_t parity) {
                if constexpr (PAIR) return mbar_wait_cluster(bar, parity, abort_flag, p.status, kWherePFull);
                return mbar_wait(bar, parity, abort_flag, p.status, kWherePFull);
            };
            // Every descriptor is "low word of the tile base + a compile-time constant" with one shared high word, so
            // an issue costs the thread a few integer instructions and the tensor pipe, not the thread, sets the pace.
            constexpr uint32_t desc_hi = umma_smem_desc_hi(1024);
            static_assert(kSlots == 2, "the selects below assume two slots");
            const uint32_t q_lo0 = umma_smem_desc_lo(smem_u32(sm.q[0]), 16), q_lo1 = umma_smem_desc_lo(smem_u32(sm.q[1]), 16);
            // stage st of a ring starts st * kStageBytes behind stage 0 (the stages are contiguous)
            const uint32_t k_lo0 = umma_smem_desc_lo(smem_u32(sm.k[0]), 16);
            const uint32_t v_lo0 = umma_smem_desc_lo(smem_u32(sm.v[0]), kPanel);
            auto issue_qk = [&](int s, int st) {
                const uint32_t qa = s ? q_lo1 : q_lo0, ka = k_lo0 + uint32_t(st) * (kStageBytes / 16u), d = tmem + uint32_t(s) * 128u;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    constexpr uint32_t unit = 16;   // descriptor addresses count 16-byte units
                    const uint32_t off = (uint32_t(kk >> 2) * kPanel + uint32_t(kk & 3) * 32u) / unit;
                    const uint32_t off_k = (uint32_t(kk >> 2) * k_panel + uint32_t(kk & 3) * 32u) / unit;
                    if (elected) {
                        if constexpr (PAIR) umma_ss_words_pair(d, qa + off, ka + off_k, desc_hi, idesc_qk, kk > 0);
                        else umma_ss_words(d, qa + off, ka + off_k, desc_hi, idesc_qk, kk > 0);
                    }
                }
                commit(&sm.s_full[s]);
            };
            // P V in two halves of four K steps: the first starts as soon as the probabilities of keys 0..63 are in
            // tensor memory, while the score-mod warps still work on keys 64..127.
            // Where P sits: the one-warp-per-row layout packs all 128 keys into the first 64 score columns; in the
            // column-split layout each half writes onto the first 32 columns of its OWN 64 score columns, so that neither
            // half ever touches a column the other still has to read.
            auto issue_pv_half = [&](int s, int st, int half, bool first) {
                const uint32_t va = v_lo0 + uint32_t(st) * (kStageBytes / 16u), d = tmem + 256u + uint32_t(s) * 128u;
                const uint32_t a = tmem + uint32_t(s) * 128u + uint32_t(half) * (SPLIT ? 64u : 32u);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    const uint32_t kk = uint32_t(half) * 4u + uint32_t(k4);
                    if (elected) {
                        if constexpr (PAIR) umma_ts_words_pair(d, a + 8u * uint32_t(k4), va + kk * (2048u / 16u), desc_hi, idesc_pv, (!first) || kk > 0);
                        else umma_ts_words(d, a + 8u * uint32_t(k4), va + kk * (2048u / 16u), desc_hi, idesc_pv, (!first) || kk > 0);
                    }
                }
                if (half == 1) commit(&sm.pv_done[s]);
            };
            bool ok = true;
            // prologue: S = Q K_0^T for both slots
            for (int s = 0; s < kSlots && ok; ++s) {
                if (n_tiles[s] == 0) continue;
                ok = mbar_wait(&sm.q_full[s], 0, abort_flag, p.status, kWhereQ) &&
                     mbar_wait(&sm.k_full[0], 0, abort_flag, p.status, kWhereKFull);
                if (!ok) break;
                tc_fence_after_sync();
                issue_qk(s, 0);
            }
            if (ok && n_max > 0) commit(&sm.k_empty[0]);
            for (int j = 0; j < n_max && ok; ++j) {
                const int st = j % kSt;
                const uint32_t ph = uint32_t(j / kSt) & 1u;
                const int st_next = (j + 1) % kSt;
                const uint32_t ph_next = uint32_t((j + 1) / kSt) & 1u;
                for (int s = 0; s < kSlots && ok; ++s) {
                    if (j >= n_tiles[s]) continue;
                    ok = mbar_wait(&sm.v_full[st], ph, abort_flag, p.status, kWhereVFull);
                    FPT_TRACE(2, 31);
                    ok = ok && wait_p(&sm.p_half[s], uint32_t(j) & 1u);
                    if (!ok) break;
                    tc_fence_after_sync();
                    FPT_TRACE(2, 10 + s);            // first half of P of slot s seen
                    issue_pv_half(s, st, 0, j == 0);
                    ok = wait_p(&sm.p_full[s], uint32_t(j) & 1u);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv_half(s, st, 1, j == 0);
                    FPT_TRACE(2, 12);
                    if (j + 1 < n_tiles[s]) {
                        ok = mbar_wait(&sm.k_full[st_next], ph_next, abort_flag, p.status, kWhereKFull);
                        if (!ok) break;
                        tc_fence_after_sync();
                        FPT_TRACE(2, 13);
                        issue_qk(s, st_next);   // executes after the P V product above: same issuing thread
                        FPT_TRACE(2, 20 + s);        // both products of slot s issued
                    }
                }
                if (!ok) break;
                commit(&sm.v_empty[st]);
                if (j + 1 < n_max) commit(&sm.k_empty[st_next]);
                FPT_TRACE(2, 30);
            }
        }
      }
    } else if constexpr (SPLIT) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
      if (!skip) {
        // ------------------------------------------------------------------ score-mod warps, column-split variant
        const int sw = warp - 4;
        const int s = sw >> 3, half = (sw >> 2) & 1;
        const int row_in_tile = 32 * (warp & 3) + lane;
        const int row = m0 + s * kTileM + row_in_tile;
        const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
        const uint32_t t_s = tmem + lane_base + uint32_t(s) * 128u + uint32_t(64 * half);
        const uint32_t t_p = t_s;     // probabilities (bf16 pairs) go back onto the first 32 of this half's own score columns
        const uint32_t t_o = tmem + lane_base + 256u + uint32_t(s) * 128u + uint32_t(64 * half);
        const int n = n_tiles[s];
        const float softcap_in = p.scale / p.softcap, mul = p.softcap * kLog2e;
        const float reference = fmaxf(mul - kFixedReferenceSpan, -mul);   // small caps: exponents in [0, 2 cap*log2(e)]
        float sum_lo = 0.0f, sum_hi = 0.0f;
        bool ok = true;
        // The eight warps of the slot meet once, at the end (the two column halves add their row sums).  A bounded
        // mbarrier wait, so that a warp that gave up after a timeout cannot strand the others.
        auto slot_sync = [&](int phase) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.ld_done[s]);
            return mbar_wait(&sm.ld_done[s], uint32_t(phase) & 1u, abort_flag, p.status, kWhereSFull);
        };
        for (int j = 0; j < n && ok; ++j) {
            FPT_TRACE(s, 1);                         // start waiting for S
            ok = mbar_wait(&sm.s_full[s], uint32_t(j) & 1u, abort_flag, p.status, kWhereSFull);
            if (!ok) break;
            tc_fence_after_sync();
            FPT_TRACE(s, 2);                         // S ready
            uint32_t sr[64];
            tmem_ld_32x32b_x32(t_s, reinterpret_cast<uint32_t(&)[32]>(sr[0]));
            tmem_ld_32x32b_x32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sr[32]));
            tmem_ld_wait();
            FPT_TRACE(s, 5);                         // S in registers
            const bool diagonal = (p.causal && j == n - 1) || (j == total_tiles - 1 && (p.seq % kTileN) != 0);
            const int limit = min(p.causal ? row : 0x7fffffff, p.seq - 1);
            const int col0 = j * kTileN + 64 * half;
            uint32_t pw[32];
            if constexpr (is_sigmoid(MODE)) {
#pragma unroll
                for (int w = 0; w < 32; ++w) {
                    if constexpr (MODE == 1) pw[w] = b3_direct_select_late(scale_pack_bf16x2(sr[2 * w], sr[2 * w + 1], p.scale), p.b3);
                    else pw[w] = native_sigmoid_pair(sr[2 * w], sr[2 * w + 1], p.sigmoid_mul, p.sigmoid_add);
                }
                if (diagonal) {
#pragma unroll
                    for (int w = 0; w < 32; ++w) {
                        if (col0 + 2 * w > limit) pw[w] &= 0xffff0000u;
                        if (col0 + 2 * w + 1 > limit) pw[w] &= 0x0000ffffu;
                    }
                }
            } else {
                // Soft-capped scores live in [-cap, cap], so ONE exponent reference serves every row and every tile:
                // cap*log2(e) - 96 (or -cap*log2(e) when that is larger, which keeps small caps near 2^0).  Exponents then
                // stay within [96 - 2 cap*log2(e), 96], i.e. [-100, 96] while
                // cap*log2(e) <= 98: nothing overflows (a row sum stays below 2^96 times the sequence length) and nothing
                // underflows.  No maximum scan, no rescaling of O, and the two column halves of a row never have to agree
                // on anything before the end.
                // One pair of keys: tanh polynomial (ALU and FMA pipes), then the exponential (special-function unit), back
                // to back, so that the two bounds overlap instead of adding up.
                auto key_pair = [&](int w, auto masked) {
                    float t0, t1;
                    if constexpr (MODE == 3) {    // native twin: both the tanh and the exponential on the special-function unit
                        mul2(__uint_as_float(sr[2 * w]), __uint_as_float(sr[2 * w + 1]), softcap_in, softcap_in, t0, t1);
                        t0 = mufu_tanh(t0);
                        t1 = mufu_tanh(t1);
                    } else {
                        const uint32_t t = eval_program<kBf16, kOddSat, 4>(scale_pack_bf16x2(sr[2 * w], sr[2 * w + 1], softcap_in), p.tanh);
                        t0 = __uint_as_float(t << 16);
                        t1 = __uint_as_float(t & 0xffff0000u);
                    }
                    float a0, a1, e0, e1;
                    fma_f32x2(t0, t1, mul, -reference, a0, a1);
                    if (EMU > 0 && ((half * 32 + w) % (EMU > 0 ? EMU / 2 : 1)) < 2) {
                        exp2_full_x2<EK>(a0, a1, e0, e1);
                    } else {
                        e0 = ex2(a0);
                        e1 = ex2(a1);
                    }
                    if constexpr (decltype(masked)::value) {   // keys beyond the diagonal or the end of the sequence
                        if (col0 + 2 * w > limit) e0 = 0.0f;
                        if (col0 + 2 * w + 1 > limit) e1 = 0.0f;
                    }
                    add_f32x2(sum_lo, sum_hi, e0, e1);
                    pw[w] = Sfu<kBf16>::pack(e0, e1);
                };
                if (!diagonal) {
#pragma unroll
                    for (int w = 0; w < 32; ++w) key_pair(w, std::false_type{});
                } else {       // a branch the whole slot takes together, so that the other tiles carry no compare / select
#pragma unroll
                    for (int w = 0; w < 32; ++w) key_pair(w, std::true_type{});
                }
            }
            FPT_TRACE(s, 3);                         // probabilities computed
            tmem_st_32x32b_x32(t_p, pw);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) arrive_p(half ? &sm.p_full[s] : &sm.p_half[s]);
            FPT_TRACE(s, 4);                         // P handed over
        }
        if (ok && n > 0) {
            float inv = 1.0f, total = 1.0f;
            if constexpr (!is_sigmoid(MODE)) {       // the two column halves add their sums
                sm.xchg[s][half][row_in_tile] = sum_lo + sum_hi;
                ok = slot_sync(0);
                total = sm.xchg[s][0][row_in_tile] + sm.xchg[s][1][row_in_tile];
                inv = 1.0f / total;
            }
            ok = ok && mbar_wait(&sm.pv_done[s], uint32_t(n - 1) & 1u, abort_flag, p.status, kWherePvDone);
            if (ok) {
                tc_fence_after_sync();
                const bool real_row = row < p.seq;
                uint16_t* out_row = p.out + int64_t(b) * p.out_stride_b + int64_t(row) * p.out_stride_s +
                                    int64_t(hq) * p.out_stride_h + 64 * half;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(t_o + c * 32, v);
                    tmem_ld_wait();
                    uint4* dst = reinterpret_cast<uint4*>(out_row + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv);
                        w.y = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv);
                        w.z = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv);
                        w.w = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv);
                        if (real_row) dst[q4] = w;
                    }
                }
                if (!is_sigmoid(MODE) && p.lse && real_row && half == 0)
                    p.lse[(int64_t(b) * p.q_heads + hq) * p.seq + row] = (reference + log2f(total)) * 0.6931471805599453f;
            }
        }
      }
    } else {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
      if (!skip) {
        // ------------------------------------------------------------------ softmax / score-mod warpgroups
        const int s = (warp - 4) >> 2;
        const int row_in_tile = 32 * (warp & 3) + lane;          // tensor-memory lane owned by this thread
        const int row = m0 + s * kTileM + row_in_tile;
        const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
        const uint32_t t_s = tmem + lane_base + uint32_t(s) * 128u;
        const uint32_t t_o = tmem + lane_base + 256u + uint32_t(s) * 128u;
        const int n = n_tiles[s];
        float row_max = -INFINITY, row_sum = 0.0f;
        bool ok = true;
        const float softcap_in = p.scale / p.softcap;           // score -> tanh argument
        const float softcap_out = p.softcap * kLog2e;           // tanh -> log2-domain score
        const float plain_scale = p.scale * kLog2e;
        for (int j = 0; j < n && ok; ++j) {
            FPT_TRACE(s, 1);                         // start waiting for S
            ok = mbar_wait(&sm.s_full[s], uint32_t(j) & 1u, abort_flag, p.status, kWhereSFull);
            if (!ok) break;
            tc_fence_after_sync();
            FPT_TRACE(s, 2);                         // S ready
            // Tiles that need a mask: the causal diagonal, and the last key tile of a sequence that is not a multiple of
            // the tile size.  Both are "column > limit" with limit = min(row if causal, last key).
            const bool diagonal = (p.causal && j == n - 1) || (j == total_tiles - 1 && (p.seq % kTileN) != 0);
            const int limit = min(p.causal ? row : 0x7fffffff, p.seq - 1);
            // the whole S row: four tensor-memory loads in flight, one wait
            uint32_t sr[kTileN];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, reinterpret_cast<uint32_t(&)[32]>(sr[c * 32]));
            tmem_ld_wait();
            FPT_TRACE(s, 5);                         // S in registers
            // P goes back in two halves (keys 0..63, then 64..127), each with its own barrier, so that the first four
            // K steps of P V run while this warp still works on the second half.
            auto hand_over = [&](int half, const uint32_t (&words)[32]) {
                tmem_st_32x32b_x32(t_s + half * 32, words);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) arrive_p(half ? &sm.p_full[s] : &sm.p_half[s]);
            };
            if constexpr (is_sigmoid(MODE)) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t pw[32];
#pragma unroll
                    for (int w = 0; w < 32; ++w) {
                        const int i = half * 32 + w;
                        if constexpr (MODE == 1) {
#ifdef FPT_DIAG_SKIP_SCOREMOD       // tuning builds only: no arithmetic, to see what the rest of the pipeline sustains
                            pw[w] = sr[2 * i] ^ sr[2 * i + 1];
#else
                            const uint32_t x = scale_pack_bf16x2(sr[2 * i], sr[2 * i + 1], p.scale);
                            pw[w] = b3_direct_select_late(x, p.b3);
#endif
                        } else {
                            pw[w] = native_sigmoid_pair(sr[2 * i], sr[2 * i + 1], p.sigmoid_mul, p.sigmoid_add);
                        }
                    }
                    if (diagonal) {  // keys beyond the diagonal contribute nothing; a branch of its own, taken by
                                     // the whole slot at once, so that the other tiles carry no compare / select
#pragma unroll
                        for (int w = 0; w < 32; ++w) {
                            const int col = j * kTileN + 2 * (half * 32 + w);
                            if (col > limit) pw[w] &= 0xffff0000u;
                            if (col + 1 > limit) pw[w] &= 0x0000ffffu;
                        }
                    }
                    if (half == 1) FPT_TRACE(s, 3);  // probabilities computed
                    hand_over(half, pw);
                }
            } else {
                // val[i] * mul is the score in log2 units: val = tanh (modes 0 and 3) or the raw score (mode 2).
                const float mul = is_softcap(MODE) ? softcap_out : plain_scale;
                if constexpr (MODE == 0) {
#pragma unroll
                    for (int i = 0; i < kTileN / 2; ++i) {
                        const uint32_t x = scale_pack_bf16x2(sr[2 * i], sr[2 * i + 1], softcap_in);
                        const uint32_t t = eval_program<kBf16, kOddSat, 4>(x, p.tanh);
                        sr[2 * i] = t << 16;              // bf16 -> fp32 is a shift
                        sr[2 * i + 1] = t & 0xffff0000u;
                    }
                } else if constexpr (MODE == 3) {
#pragma unroll
                    for (int i = 0; i < kTileN / 2; ++i) {
                        float x0, x1;
                        mul2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]), softcap_in, softcap_in, x0, x1);
                        sr[2 * i] = __float_as_uint(mufu_tanh(x0));
                        sr[2 * i + 1] = __float_as_uint(mufu_tanh(x1));
                    }
                }
                if (diagonal) {
#pragma unroll
                    for (int i = 0; i < kTileN; ++i)
                        if (j * kTileN + i > limit) sr[i] = 0xff800000u;  // -inf
                }
                // Row maximum of the tile (three-input max on the ALU pipe, which has room beside the exponentials).
                // The reference point of the exponentials moves only when the maximum grew by more than 2^8 (lazy
                // rescale); the decision is taken for the whole warp because the tensor-memory accesses of the
                // rescale are warp-wide instructions.
                float m3 = __uint_as_float(sr[0]);
#pragma unroll
                for (int i = 1; i + 1 < kTileN; i += 2)
                    m3 = max3(m3, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
                const float tile_max = fmaxf(m3, __uint_as_float(sr[kTileN - 1])) * mul;
                const bool move = tile_max > row_max + kRescaleThreshold;     // always true on the first tile
                if (__any_sync(0xffffffffu, move)) {
                    const float f = move ? ex2(row_max - tile_max) : 1.0f;
                    if (move) row_max = tile_max;
                    row_sum *= f;
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            uint32_t v[32];
                            tmem_ld_32x32b_x32(t_o + c * 32, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
                            tmem_st_32x32b_x32(t_o + c * 32, v);
                        }
                        tmem_st_wait();
                    }
                }
                float sum_lo = 0.0f, sum_hi = 0.0f;
                const float neg_max = -row_max;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t pw[32];
#pragma unroll
                    for (int w = 0; w < 32; ++w) {
                        const int i = half * 32 + w;
                        float a0, a1;
                        fma_f32x2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]), mul, neg_max, a0, a1);
                        float e0, e1;
                        if (EMU > 0 && (i % (EMU > 0 ? EMU / 2 : 1)) < 2) {
                            exp2_full_x2<EK>(a0, a1, e0, e1);   // FMA pipe: keys 2i, 2i+1 fall in the routed four of their group
                        } else {
                            e0 = ex2(a0);                    // special-function unit
                            e1 = ex2(a1);
                        }
                        add_f32x2(sum_lo, sum_hi, e0, e1);
                        pw[w] = Sfu<kBf16>::pack(e0, e1);
                    }
                    if (half == 1) FPT_TRACE(s, 3);  // probabilities computed
                    hand_over(half, pw);
                }
                row_sum += sum_lo + sum_hi;
            }
            FPT_TRACE(s, 4);                         // P handed over
        }
        if (ok && n > 0) {
            ok = mbar_wait(&sm.pv_done[s], uint32_t(n - 1) & 1u, abort_flag, p.status, kWherePvDone);
            if (ok) {
                tc_fence_after_sync();
                const float inv = is_sigmoid(MODE) ? 1.0f : 1.0f / row_sum;
                const bool real_row = row < p.seq;       // rows of a ragged last tile beyond the sequence are dropped
                uint16_t* out_row = p.out + int64_t(b) * p.out_stride_b + int64_t(row) * p.out_stride_s +
                                    int64_t(hq) * p.out_stride_h;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(t_o + c * 32, v);
                    tmem_ld_wait();
                    uint4* dst = reinterpret_cast<uint4*>(out_row + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv);
                        w.y = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv);
                        w.z = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv);
                        w.w = Sfu<kBf16>::pack(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv);
                        if (real_row) dst[q4] = w;
                    }
                }
                if (!is_sigmoid(MODE) && p.lse && real_row)
                    p.lse[(int64_t(b) * p.q_heads + hq) * p.seq + row] = (row_max + log2f(row_sum)) * 0.6931471805599453f;
            }
        }
      }
    }
    tc_fence_before_sync();
    if constexpr (PAIR) {
        __syncwarp();
        cluster_sync_all();        // neither CTA leaves while the other can still reach its barriers or memory
        if (warp == 1) tmem_dealloc_pair(tmem, 512);
    } else {
        __syncthreads();
        if (warp == 1) tmem_dealloc(tmem, 512);
    }
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_attention_fwd_routed(void* out, void* lse, const void* q, const void* k, const void* v, int64_t batch,
                                        int64_t seq, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                        const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                        const int64_t* out_strides, int mode, int causal, float scale, float softcap,
                                        int log2_n, int exp2_emu_backend, int exp2_emu_freq, void* status,
                                        fpt_stream_t stream) {
    if (!out || !q || !k || !v || !status || !q_strides || !k_strides || !v_strides || !out_strides)
        return FPT_ERR_NULL_POINTER;
    if (batch <= 0 || seq <= 0 || q_heads <= 0 || kv_heads <= 0) return FPT_ERR_BAD_SIZE;
    if (head_dim != kHeadDim || q_heads % kv_heads != 0) return FPT_ERR_UNSUPPORTED_SHAPE;
    if (batch > 65535 || q_heads > 0x7fffffff || seq > 0x3fffffff) return FPT_ERR_BAD_SIZE;
    if (mode < FPT_ATTN_SOFTCAP_TANH || mode > FPT_ATTN_SIGMOID_NATIVE) return FPT_ERR_BAD_ENUM;
    const bool softcap_family = mode == FPT_ATTN_SOFTCAP_TANH || mode == FPT_ATTN_SOFTCAP_NATIVE;
    const bool sigmoid_family = mode == FPT_ATTN_SIGMOID_DIRECT || mode == FPT_ATTN_SIGMOID_NATIVE;
    if (softcap_family && !(softcap > 0.0f)) return FPT_ERR_BAD_SIZE;
    if (sigmoid_family && (log2_n < 1 || log2_n > 24)) return FPT_ERR_BAD_SIZE;
    if (exp2_emu_freq != 0 && exp2_emu_freq != 8 && exp2_emu_freq != 12 && exp2_emu_freq != 16 && exp2_emu_freq != 32)
        return FPT_ERR_BAD_ENUM;
    // routing exists where an exponential exists and a polynomial is asked for: not in the sigmoid modes, not in the
    // all-native soft-cap twin
    if ((sigmoid_family || mode == FPT_ATTN_SOFTCAP_NATIVE) && exp2_emu_freq != 0) return FPT_ERR_BAD_ENUM;
    if (exp2_emu_backend < FPT_EXP2_FULL_D3 || exp2_emu_backend > FPT_EXP2_FULL_PWL2_SAFE_F16) return FPT_ERR_BAD_ENUM;
    if (exp2_emu_backend != FPT_EXP2_FULL_D3 && exp2_emu_freq != 0 && mode != FPT_ATTN_SOFTMAX) return FPT_ERR_BAD_ENUM;
    if (reinterpret_cast<uintptr_t>(out) & 15u) return FPT_ERR_MISALIGNED;
    for (int i = 0; i < 3; ++i)
        if ((out_strides[i] * 2) & 15) return FPT_ERR_MISALIGNED;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;

    // strides arrive as (batch, seq, head) in elements; the tensor maps want (seq, head, batch) in bytes
    auto make_map = [&](CUtensorMap* map, const void* base, const int64_t* st, int64_t heads) {
        const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(seq), uint64_t(heads), uint64_t(batch)};
        const uint64_t strides[3] = {uint64_t(st[1]) * 2, uint64_t(st[2]) * 2, uint64_t(st[0]) * 2};
        return make_tensor_map_bf16_4d(map, base, dims, strides, kTileM);
    };
    CUtensorMap map_q, map_k, map_v, map_kh;
    if (int rc = make_map(&map_q, q, q_strides, q_heads)) return rc;
    if (int rc = make_map(&map_k, k, k_strides, kv_heads)) return rc;
    if (int rc = make_map(&map_v, v, v_strides, kv_heads)) return rc;
    {   // the K map with a box of 64 keys: what one CTA of a pair loads of a key tile
        const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(seq), uint64_t(kv_heads), uint64_t(batch)};
        const uint64_t strides[3] = {uint64_t(k_strides[1]) * 2, uint64_t(k_strides[2]) * 2, uint64_t(k_strides[0]) * 2};
        if (int rc = make_tensor_map_bf16_4d(&map_kh, k, dims, strides, kTileN / 2)) return rc;
    }

    AttnParams p{};
    p.out = static_cast<uint16_t*>(out);
    p.lse = static_cast<float*>(lse);
    p.out_stride_b = out_strides[0];
    p.out_stride_s = out_strides[1];
    p.out_stride_h = out_strides[2];
    p.batch = int(batch); p.seq = int(seq); p.q_heads = int(q_heads); p.kv_heads = int(kv_heads);
    p.mode = mode; p.causal = causal ? 1 : 0;
    p.scale = scale; p.softcap = softcap;
    p.status = static_cast<uint32_t*>(status);
    const ProgramRow* tanh_row = find_program(FPT_FN_TANH, FPT_FWD, 4, FPT_BF16, FPT_SRC_CURRENT);
    if (!tanh_row || tanh_row->shape != kOddSat) return FPT_ERR_UNKNOWN_PROGRAM;
    p.tanh = program_words(*tanh_row);
    p.b3 = b3_words(mode == FPT_ATTN_SIGMOID_DIRECT ? log2_n : 12);
    p.sigmoid_mul = -scale * kLog2e;          // 1 / (1 + 2^(log2 n - s*scale*log2 e)) = sigmoid(s*scale - ln n)
    p.sigmoid_add = float(log2_n);

    const size_t smem = sizeof(AttnSmem) + 1024;
    static_assert(sizeof(AttnSmem) + 1024 <= 227 * 1024, "shared memory budget");
    const int n_qblocks = int((seq + kSlots * kTileM - 1) / (kSlots * kTileM));
    // Measured: with a causal mask heads fastest wins by 3-20 % (blocks that run together have the same length).  Without
    // a mask isolated launches run alike in either order (B=2, S=16384, 32 heads: within 1 %), but heads fastest streams the
    // K / V of every head at once (537 MB there, against 126 MB of L2: 30 GB of re-reads per launch), and in a run long
    // enough to meet the power cap that traffic costs clock: rows fastest 1020-1100 against 885-990 TFLOP/s.  So: rows
    // fastest when nothing is masked and K and V together exceed 64 MB, heads fastest otherwise.
    const int raster = fpt::tuning_attention_raster();
    const int64_t kv_bytes = 2 * batch * kv_heads * seq * head_dim * 2;
    p.rows_fastest = raster >= 0 ? raster : (!causal && kv_bytes > (int64_t(64) << 20) ? 1 : 0);
    // Pairs of CTAs (clusters of two along x) need two blocks that walk the same K / V in step: two query heads of one
    // K / V group (heads on x, even group size: they also share their causal length), or two neighbouring row blocks of one
    // head where no mask makes their lengths differ (rows on x, whole blocks only).
    bool pair = false;
    if (fpt::tuning_attention_cta_pair() == 1 && exp2_emu_freq == 0) {
        const bool heads_pair = (q_heads / kv_heads) % 2 == 0;
        const bool rows_pair = !causal && n_qblocks % 2 == 0 && seq % (kSlots * kTileM) == 0;
        if (heads_pair && (raster != 1 || !rows_pair)) { pair = true; p.rows_fastest = 0; }
        else if (rows_pair) { pair = true; p.rows_fastest = 1; }
    }
    const dim3 grid = p.rows_fastest ? dim3{unsigned(n_qblocks), unsigned(q_heads), unsigned(batch)}
                                     : dim3{unsigned(q_heads), unsigned(n_qblocks), unsigned(batch)};
    auto launch = [&](auto kernel, int threads) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
        kernel<<<grid, threads, smem, stream>>>(map_q, map_k, map_v, map_kh, p);
        return cuda_status(cudaGetLastError());
    };
    auto launch_pair = [&](auto kernel, int threads) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
        cudaLaunchConfig_t config{};
        config.gridDim = grid;
        config.blockDim = dim3{unsigned(threads), 1, 1};
        config.dynamicSmemBytes = smem;
        config.stream = reinterpret_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attribute{};
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = 2;
        attribute.val.clusterDim.y = 1;
        attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        return cuda_status(cudaLaunchKernelEx(&config, kernel, map_q, map_k, map_v, map_kh, p));
    };
    if (pair) {
        const bool split_pair = softcap_family && softcap * kLog2e <= kFixedReferenceLimit && fpt::tuning_attention_split() >= 1;
        switch (mode) {
            case FPT_ATTN_SOFTCAP_TANH:
                return split_pair ? launch_pair(attention_fwd_kernel<0, 0, true, kExp2FullD3, true>, kThreadsSplit)
                                  : launch_pair(attention_fwd_kernel<0, 0, false, kExp2FullD3, true>, kThreads);
            case FPT_ATTN_SIGMOID_DIRECT: return launch_pair(attention_fwd_kernel<1, 0, false, kExp2FullD3, true>, kThreads);
            case FPT_ATTN_SOFTMAX: return launch_pair(attention_fwd_kernel<2, 0, false, kExp2FullD3, true>, kThreads);
            case FPT_ATTN_SOFTCAP_NATIVE:
                return split_pair ? launch_pair(attention_fwd_kernel<3, 0, true, kExp2FullD3, true>, kThreadsSplit)
                                  : launch_pair(attention_fwd_kernel<3, 0, false, kExp2FullD3, true>, kThreads);
            default: return launch_pair(attention_fwd_kernel<4, 0, false, kExp2FullD3, true>, kThreads);
        }
    }
    // The column-split variant pays where the score-mod is instruction-heavy and needs no per-tile row reduction: the
    // soft-capped mode while cap * log2(e) stays within the range its fixed exponent reference covers (measured +15..28 %
    // since its tanh and exponential run back to back per key pair).  The sigmoid mode also qualifies but measures no
    // faster with it (0.98..1.0x), so it keeps one thread per row unless the tuning key asks for the split layout.
    const int split_tuning = fpt::tuning_attention_split();
    const bool split = softcap_family && softcap * kLog2e <= kFixedReferenceLimit && split_tuning >= 1;
    if (mode == FPT_ATTN_SIGMOID_DIRECT)
        return split_tuning >= 2 ? launch(attention_fwd_kernel<1, 0, true>, kThreadsSplit) : launch(attention_fwd_kernel<1, 0, false>, kThreads);
    if (mode == FPT_ATTN_SIGMOID_NATIVE) return launch(attention_fwd_kernel<4, 0, false>, kThreads);
    if (mode == FPT_ATTN_SOFTCAP_NATIVE)
        return split ? launch(attention_fwd_kernel<3, 0, true>, kThreadsSplit) : launch(attention_fwd_kernel<3, 0, false>, kThreads);
    const bool softcap_mode = mode == FPT_ATTN_SOFTCAP_TANH;
    if (softcap_mode && split) {
        switch (exp2_emu_freq) {
            case 0: return launch(attention_fwd_kernel<0, 0, true>, kThreadsSplit);
            case 8: return launch(attention_fwd_kernel<0, 8, true>, kThreadsSplit);
            case 12: return launch(attention_fwd_kernel<0, 12, true>, kThreadsSplit);
            case 16: return launch(attention_fwd_kernel<0, 16, true>, kThreadsSplit);
            default: return launch(attention_fwd_kernel<0, 32, true>, kThreadsSplit);
        }
    }
    // plain soft-max with a routed software exponential other than the cubic
    auto routed_softmax = [&](auto kind) {
        constexpr int EK = decltype(kind)::value;
        switch (exp2_emu_freq) {
            case 8: return launch(attention_fwd_kernel<2, 8, false, EK>, kThreads);
            case 12: return launch(attention_fwd_kernel<2, 12, false, EK>, kThreads);
            case 16: return launch(attention_fwd_kernel<2, 16, false, EK>, kThreads);
            default: return launch(attention_fwd_kernel<2, 32, false, EK>, kThreads);
        }
    };
    if (!softcap_mode && exp2_emu_freq != 0) {
        if (exp2_emu_backend == FPT_EXP2_FULL_PWL2) return routed_softmax(IC<kExp2FullPwl2>{});
        if (exp2_emu_backend == FPT_EXP2_FULL_D2_SAFE) return routed_softmax(IC<kExp2FullD2Safe>{});
        if (exp2_emu_backend == FPT_EXP2_FULL_PWL2_SAFE_F16) return routed_softmax(IC<kExp2FullPwl2SafeF16>{});
    }
    switch (exp2_emu_freq) {
        case 0: return softcap_mode ? launch(attention_fwd_kernel<0, 0, false>, kThreads) : launch(attention_fwd_kernel<2, 0, false>, kThreads);
        case 8: return softcap_mode ? launch(attention_fwd_kernel<0, 8, false>, kThreads) : launch(attention_fwd_kernel<2, 8, false>, kThreads);
        case 12: return softcap_mode ? launch(attention_fwd_kernel<0, 12, false>, kThreads) : launch(attention_fwd_kernel<2, 12, false>, kThreads);
        case 16: return softcap_mode ? launch(attention_fwd_kernel<0, 16, false>, kThreads) : launch(attention_fwd_kernel<2, 16, false>, kThreads);
        default: return softcap_mode ? launch(attention_fwd_kernel<0, 32, false>, kThreads) : launch(attention_fwd_kernel<2, 32, false>, kThreads);
    }
}

extern "C" int fpt_attention_fwd(void* out, void* lse, const void* q, const void* k, const void* v, int64_t batch,
                                 int64_t seq, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                 const int64_t* out_strides, int mode, int causal, float scale, float softcap, int log2_n,
                                 void* status, fpt_stream_t stream) {
    return fpt_attention_fwd_routed(out, lse, q, k, v, batch, seq, q_heads, kv_heads, head_dim, q_strides, k_strides,
                                    v_strides, out_strides, mode, causal, scale, softcap, log2_n, FPT_EXP2_FULL_D3, 0,
                                    status, stream);
}
