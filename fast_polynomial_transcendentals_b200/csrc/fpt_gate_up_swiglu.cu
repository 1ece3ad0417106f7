// Gate / up projection with the SwiGLU applied in the epilogue, for sm_100a: out = swish(x Wg^T) * (x Wu^T) without the
// [rows, 2 hidden] intermediate ever reaching memory.  Dense (one weight pair) and grouped (expert-sorted rows, one
// weight pair per group) in one kernel.
//
// Persistent CTAs, one per SM, each walking tiles of (128 x HALVES) rows x 128 hidden columns.  128 rows of a tile own
// ONE accumulator of 128 x 256 fp32 in tensor memory: columns 0..127 are the gate product, 128..255 the up product of
// the same hidden columns, so that one tcgen05.mma of shape 128 x 256 x 16 feeds both and the epilogue finds a gate
// value and its up value in the same lane.
//   warp 0      TMA producer: x tile [128 HALVES x 64] and the two weight tiles [128 x 64] per K block into a ring
//   warp 1      tcgen05.mma issuer, converged warp with an elected lane (both operands K-major from shared memory, 128-byte swizzle)
//   warp 2      allocates tensor memory (512 columns = two accumulators)
//   warps 4..   epilogue, four warps per accumulator: thread = one row; fp32 -> bf16 (round to nearest even, what a
//               separate GEMM would have stored), then the same packed polynomial program as fpt_swish_mul, then
//               16-byte stores
// HALVES = 1 (grouped problems: ragged groups waste less of a 128-row tile): the two accumulators alternate, the epilogue
// of a tile runs under the products of the next one; 4-stage ring.
// HALVES = 2 (dense problems): both accumulators belong to one tile of 256 rows whose two halves share every weight
// tile, which takes a third off the bytes that have to arrive per product (64 instead of 96 KiB per 2 x 128 x 256 x 64)
// -- in a loop long enough to meet the power cap the form that moves fewer bytes per product is the faster one -- at
// the price of an epilogue that overlaps only with the loads of the next tile; 3-stage ring of 64 KiB.
// A third form runs the 256-row tile on a PAIR of CTAs (gate_up_swiglu_pair_kernel below).
// In every form the result equals fpt_swish_mul_packed applied to this kernel's own raw [gate | up] output bit for bit
// (epilogue = FPT_GATE_UP_RAW writes that output).
// Tile order: bands of 4096 rows; inside a band the hidden tile is the slow index, so that the CTAs running together
// share a few weight panels and the band's rows stay in L2 (measured at 16384 x 4096 -> 14336 under the power cap: bands
// of 1024 / 2048 / 4096 / 8192 / 16384 rows give 0.93 / 0.95 / 1 / 0.93 / 0.83 of the best rate).  Groups are bands of
// their own (their rows use other weights).
// Every mbarrier wait is bounded; on a timeout the CTA records where it stopped and unwinds.
#include <algorithm>
#include <type_traits>

#include "fpt_common.h"
#include "fpt_programs.h"
#include "fpt_sm100.cuh"

namespace fpt {
namespace {

using namespace sm100;

constexpr int kRowsPerHalf = 128;
constexpr int kHiddenPerTile = 128;
constexpr int kBlockK = 64;
#ifndef FPT_GATE_UP_BAND_ROWS
#define FPT_GATE_UP_BAND_ROWS 4096
#endif
// Tuning builds only (-DFPT_GATE_UP_DIAG=n): 1 leaves out the epilogue's work, 2 the loads (the products run on whatever
// shared memory holds), 3 the products; each shows what the other two sustain alone.  Results are then meaningless.
#ifndef FPT_GATE_UP_DIAG
#define FPT_GATE_UP_DIAG 0
#endif
constexpr int kBandRows = FPT_GATE_UP_BAND_ROWS;   // rows per band
constexpr int kMaxGroups = 256;
constexpr uint32_t kXHalfBytes = kRowsPerHalf * 128;   // 128 rows x 64 bf16
constexpr uint32_t kWBytes = 2 * kHiddenPerTile * 128;
constexpr int kMaxThreads = 384;

// rows of every group and the number of tiles before it, built by the whole CTA at kernel start
struct TileTable {
    int32_t group_begin[kMaxGroups], group_end[kMaxGroups];
    int32_t tile_prefix[kMaxGroups + 1];
    int32_t warp_total[kMaxThreads / 32];
};

template <int HALVES>
struct GateUpSmem {
    static constexpr int kRing = 192 * 1024 / int(HALVES * kXHalfBytes + kWBytes);
    alignas(1024) uint8_t x[kRing][HALVES * kXHalfBytes];
    alignas(1024) uint8_t w[kRing][kWBytes];       // rows 0..127 gate weights, 128..255 up weights
    alignas(8) uint64_t full[kRing];
    uint64_t empty[kRing];
    uint64_t acc_full[2], acc_empty[2];
    TileTable table;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

struct GateUpParams {
    uint16_t* out;
    const int32_t* group_ends;     // device, cumulative row counts per group, or null (one group of all rows)
    int64_t out_ld;
    int rows, hidden, groups;
    int hidden_tiles, k_blocks;
    uint32_t* status;
};

enum : uint32_t { kGuEmpty = 1, kGuFull, kGuAccEmpty, kGuAccFull };

struct Tile {
    int row0, row_end, hidden_tile, group;
};

// tile index -> coordinates; every role decodes the same sequence
template <int ROWS_PER_TILE>
__device__ __forceinline__ Tile decode_tile(const TileTable& tb, const GateUpParams& p, int tile) {
    constexpr int kBand = kBandRows / ROWS_PER_TILE;
    int lo = 0, hi = p.groups - 1;
    while (lo < hi) {                               // last group whose prefix is <= tile
        const int mid = (lo + hi + 1) >> 1;
        if (tb.tile_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const int g = lo;
    const int begin = tb.group_begin[g], end = tb.group_end[g];
    const int row_tiles = (end - begin + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
    const int r = tile - tb.tile_prefix[g];
    const int per_band = kBand * p.hidden_tiles;
    const int band = r / per_band, r2 = r - band * per_band;
    const int in_band = min(kBand, row_tiles - band * kBand);
    const int hidden_tile = r2 / in_band, row_tile = band * kBand + (r2 - hidden_tile * in_band);
    return Tile{begin + row_tile * ROWS_PER_TILE, end, hidden_tile, g};
}

// Called by every thread of the CTA (at least 256 of them, one per possible group); contains a __syncthreads, and the
// caller synchronises once more before the table is read.
template <int ROWS_PER_TILE>
__device__ __forceinline__ void build_tile_table(TileTable& tb, const GateUpParams& p) {
    const int g = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int begin = 0, end = 0;
    if (g < p.groups) {
        if (p.group_ends) {
            begin = g ? p.group_ends[g - 1] : 0;
            end = p.group_ends[g];
        } else {
            end = p.rows;
        }
        begin = min(max(begin, 0), p.rows);
        end = min(max(end, begin), p.rows);
        tb.group_begin[g] = begin;
        tb.group_end[g] = end;
    }
    const int tiles = (end - begin + ROWS_PER_TILE - 1) / ROWS_PER_TILE * p.hidden_tiles;
    int scan = tiles;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, scan, off);
        if (lane >= off) scan += other;
    }
    if (lane == 31) tb.warp_total[warp] = scan;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += tb.warp_total[w];
    if (g < p.groups) tb.tile_prefix[g + 1] = before + scan;
    if (g == 0) tb.tile_prefix[0] = 0;
}

// One warp's share of an accumulator (its 32 lanes = 32 rows, 128 hidden columns): fp32 -> bf16, the SwiGLU program (or
// the two products as they are), 16-byte stores.  `t_acc` is the accumulator's tensor-memory address with the warp's
// lane offset; gate values sit in columns 0..127, up values in 128..255.
template <class Op>
__device__ __forceinline__ void epilogue_rows(const Op& op, const GateUpParams& p, uint32_t t_acc, uint16_t* out_row, bool valid);

struct RawEpilogue {};

template <class Op>
__device__ __forceinline__ void epilogue_rows(const Op& op, const GateUpParams& p, uint32_t t_acc, uint16_t* out_row, bool valid) {
#if FPT_GATE_UP_DIAG != 1
#pragma unroll 1
    for (int c = 0; c < kHiddenPerTile / 32; ++c) {
        uint32_t g[32], u[32];
        tmem_ld_32x32b_x32(t_acc + uint32_t(c) * 32u, g);
        tmem_ld_32x32b_x32(t_acc + 128u + uint32_t(c) * 32u, u);
        tmem_ld_wait();
        uint32_t gw[16], uw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            gw[i] = Sfu<kBf16>::pack(__uint_as_float(g[2 * i]), __uint_as_float(g[2 * i + 1]));
            uw[i] = Sfu<kBf16>::pack(__uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]));
        }
        if constexpr (std::is_same<Op, RawEpilogue>::value) {
            if (valid) {
                uint4* dg = reinterpret_cast<uint4*>(out_row + c * 32);
                uint4* du = reinterpret_cast<uint4*>(out_row + p.hidden + c * 32);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    dg[q] = make_uint4(gw[4 * q], gw[4 * q + 1], gw[4 * q + 2], gw[4 * q + 3]);
                    du[q] = make_uint4(uw[4 * q], uw[4 * q + 1], uw[4 * q + 2], uw[4 * q + 3]);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t in[2] = {gw[i], uw[i]};
                uint32_t o[1];
                op.apply(in, o);
                gw[i] = o[0];
            }
            if (valid) {
                uint4* dst = reinterpret_cast<uint4*>(out_row + c * 32);
#pragma unroll
                for (int q = 0; q < 4; ++q) dst[q] = make_uint4(gw[4 * q], gw[4 * q + 1], gw[4 * q + 2], gw[4 * q + 3]);
            }
        }
    }
#endif
}

template <class Op, int HALVES>
__global__ void __launch_bounds__(128 + 128 * HALVES, 1)
gate_up_swiglu_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                      const __grid_constant__ CUtensorMap map_wu, const GateUpParams p, const Op op) {
    using Smem = GateUpSmem<HALVES>;
    constexpr int kRing = Smem::kRing, kRowsPerTile = kRowsPerHalf * HALVES;
    constexpr uint32_t kXBytes = HALVES * kXHalfBytes;
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile uint32_t* abort_flag = &sm.abort_flag;

    build_tile_table<kRowsPerTile>(sm.table, p);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRing; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sm.acc_full[a], 1);
            mbar_init(&sm.acc_empty[a], 4);        // one arrive per epilogue warp
        }
        sm.abort_flag = *reinterpret_cast<volatile uint32_t*>(p.status) != 0u ? 1u : 0u;
        mbar_fence_init();
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_wg);
        tma_prefetch_descriptor(&map_wu);
    }
    if (warp == 2) {
        tmem_alloc(&sm.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const int total_tiles = sm.table.tile_prefix[p.groups];
    const bool skip = sm.abort_flag != 0u;

    // Accumulators: HALVES = 1 alternates them (tile `local` uses accumulator local & 1 for the (local >> 1)-th time);
    // HALVES = 2 gives accumulator h to rows 128 h .. 128 h + 127 of every tile.
    if (skip) {
        // a CTA that starts after another one reported a timeout does nothing
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const Tile t = decode_tile<kRowsPerTile>(sm.table, p, tile);
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % kRing, use = it / kRing;
                    if (use > 0) ok = mbar_wait(&sm.empty[s], (use - 1u) & 1u, abort_flag, p.status, kGuEmpty);
                    if (!ok) break;
#if FPT_GATE_UP_DIAG == 2
                    mbar_arrive(&sm.full[s]);
#else
                    mbar_arrive_expect_tx(&sm.full[s], kXBytes + kWBytes);
                    tma_load_4d(sm.x[s], &map_x, &sm.full[s], kb * kBlockK, t.row0, 0, 0);
                    tma_load_4d(sm.w[s], &map_wg, &sm.full[s], kb * kBlockK, t.hidden_tile * kHiddenPerTile, t.group, 0);
                    tma_load_4d(sm.w[s] + kWBytes / 2, &map_wu, &sm.full[s], kb * kBlockK, t.hidden_tile * kHiddenPerTile,
                                t.group, 0);
#endif
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ tcgen05.mma issuer
        // The whole warp runs the loop (waits included) and one elected lane issues: see elect_one().
        {
            const bool elected = elect_one();
            constexpr uint32_t idesc = umma_idesc_bf16(kRowsPerHalf, 2 * kHiddenPerTile, 0, 0);
            constexpr uint32_t desc_hi = umma_smem_desc_hi(1024);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                for (int kb = 0; kb < p.k_blocks && ok; ++kb, ++it) {
                    const uint32_t s = it % kRing, use_s = it / kRing;
                    ok = mbar_wait(&sm.full[s], use_s & 1u, abort_flag, p.status, kGuFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t x_lo = umma_smem_desc_lo(smem_u32(sm.x[s]), 16);
                    const uint32_t w_lo = umma_smem_desc_lo(smem_u32(sm.w[s]), 16);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        const uint32_t a = HALVES == 1 ? (local & 1u) : uint32_t(h);
                        const uint32_t use = HALVES == 1 ? (local >> 1) : local;
                        if (kb == 0 && use > 0) {       // the epilogue of this accumulator's previous tile has read it
                            ok = mbar_wait(&sm.acc_empty[a], (use - 1u) & 1u, abort_flag, p.status, kGuAccEmpty);
                            if (!ok) break;
                            tc_fence_after_sync();
                        }
                        const uint32_t d = tmem + a * 256u, xh = x_lo + uint32_t(h) * (kXHalfBytes / 16u);
#if FPT_GATE_UP_DIAG != 3
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / 16; ++k)  // 32 bytes along the swizzled row per K step of 16
                            if (elected) umma_ss_words(d, xh + 2u * k, w_lo + 2u * k, desc_hi, idesc, (kb > 0 || k > 0) ? 1u : 0u);
#endif
                    }
                    if (!ok) break;
                    if (elected) umma_commit(&sm.empty[s]);
                }
                if (ok) {
                    if constexpr (HALVES == 1) {
                        if (elected) umma_commit(&sm.acc_full[local & 1u]);
                    } else {
                        if (elected) umma_commit(&sm.acc_full[0]);
                        if (elected) umma_commit(&sm.acc_full[1]);
                    }
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue
        const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
        const int half = (warp - 4) >> 2;              // 0 when HALVES = 1
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const Tile t = decode_tile<kRowsPerTile>(sm.table, p, tile);
            const uint32_t a = HALVES == 1 ? (local & 1u) : uint32_t(half);
            const uint32_t use = HALVES == 1 ? (local >> 1) : local;
            ok = mbar_wait(&sm.acc_full[a], use & 1u, abort_flag, p.status, kGuAccFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int row = t.row0 + half * kRowsPerHalf + 32 * (warp & 3) + lane;
            const bool valid = row < t.row_end;
            const uint32_t t_acc = tmem + lane_base + a * 256u;
            uint16_t* out_row = p.out + int64_t(row) * p.out_ld + t.hidden_tile * kHiddenPerTile;
            epilogue_rows(op, p, t_acc, out_row, valid);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.acc_empty[a]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem, 512);
}

// ---- the same tile of 256 rows on a PAIR of CTAs (cta_group::2) -----------------------------------------------------
// The two CTAs of a cluster of two take 128 rows each.  The leading CTA (rank 0) loads the gate weight tile, the other
// the up weight tile, each into the same shared-memory offset, and ONE tcgen05.mma.cta_group::2 of shape 256 x 256 x 16,
// issued by the leading CTA, reads A from both (their own rows) and the two halves of B's N rows from both, and leaves
// every CTA its 128 x 256 [gate | up] accumulator in its own tensor memory.  Per CTA and K block 32 KiB arrive (as with
// 256-row tiles on one CTA) but only 16 + 16 KiB are read per product, the ring is six deep and the two accumulators
// alternate again, so the epilogue runs under the next tile's products.
// Hand-overs: the loads of both CTAs complete on the leading CTA's `full` barrier (cp.async.bulk.tensor ... cta_group::2
// with the barrier's shared::cluster address; the barrier expects the bytes of both); the issuer's commits reach `empty`
// and `acc_full` in both CTAs at once (tcgen05.commit ... multicast); the epilogue warps of both CTAs arrive on the
// leading CTA's `acc_empty` (8 arrivals, the other CTA's through a remote arrive).
// A first form let each CTA's loads complete on its own barrier and had a thread of the other CTA pass that on with
// mbarrier.arrive.release.cluster: it ran at HALF speed, because a releasing remote arrive waits for every bulk load
// still in flight into its CTA, which empties the ring (a relaxed arrive restored the speed; the direct form needs none).
// WIDE = 2 gives the pair TWO hidden tiles per row tile (a 256 x 256 output tile, [gate | up] accumulators for both in the
// 512 columns of tensor memory): x arrives once for both, which takes another quarter off the bytes per product (48
// instead of 64 KiB per K block and CTA, for twice the products); the ring is four stages of 48 KiB and the epilogue (eight
// warps, one accumulator per four) overlaps only with the loads of the next tile.  Needs an even number of hidden tiles.
// Measured SLOWER than one hidden tile per row tile (16384 x 4096 -> 14336: 1362 against 1477 TFLOP/s back to back, 1521
// against 1550 isolated): the alternating accumulators and the deeper ring are worth more than the bytes.  Opt-in.
constexpr uint32_t kPairColumns = 512;

template <int WIDE>
struct GateUpPairSmem {
    static constexpr int kRing = 192 * 1024 / int(kXHalfBytes * (1 + WIDE));
    alignas(1024) uint8_t x[kRing][kXHalfBytes];
    alignas(1024) uint8_t w[kRing][WIDE * kXHalfBytes];    // rank 0: 128 gate weight rows per hidden tile; rank 1: up weight rows
    alignas(8) uint64_t full[kRing];
    uint64_t empty[kRing];
    uint64_t acc_full[2], acc_empty[2];                    // acc_empty used in the leading CTA
    TileTable table;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

template <class Op, int WIDE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128 + 128 * WIDE, 1)
gate_up_swiglu_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                           const __grid_constant__ CUtensorMap map_wu, const GateUpParams p, const Op op) {
    constexpr int kRowsPerTile = 2 * kRowsPerHalf;
    extern __shared__ uint8_t smem_raw[];
    // the same offsets in both CTAs: the dynamic shared memory of both starts at the same address
    using Smem = GateUpPairSmem<WIDE>;
    constexpr int kPairRing = Smem::kRing;
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    volatile uint32_t* abort_flag = &sm.abort_flag;

    build_tile_table<kRowsPerTile>(sm.table, p);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairRing; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sm.acc_full[a], 1);
            mbar_init(&sm.acc_empty[a], 8);        // four epilogue warps in each CTA
        }
        sm.abort_flag = *reinterpret_cast<volatile uint32_t*>(p.status) != 0u ? 1u : 0u;
        mbar_fence_init();
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(rank == 0 ? &map_wg : &map_wu);
    }
    if (warp == 2) {
        tmem_alloc_pair(&sm.tmem_base, kPairColumns);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();                             // barriers of both CTAs initialised before anyone arrives remotely
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const int total_tiles = sm.table.tile_prefix[p.groups];
    const bool skip = sm.abort_flag != 0u;
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
#ifdef FPT_GATE_UP_PAIR_DEBUG
    if (threadIdx.x == 0 && blockIdx.x < 2) p.status[4 + rank] = tmem + 1u;   // tuning builds: the address each CTA was given
#endif

    if (skip) {
        // a CTA that starts after another one reported a timeout does nothing
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            const CUtensorMap* map_w = rank == 0 ? &map_wg : &map_wu;
            uint32_t it = 0;
            bool ok = true;
            for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
                const Tile t = decode_tile<kRowsPerTile>(sm.table, p, tile);
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % kPairRing, use = it / kPairRing;
                    if (use > 0) ok = mbar_wait(&sm.empty[s], (use - 1u) & 1u, abort_flag, p.status, kGuEmpty);
                    if (!ok) break;
#if FPT_GATE_UP_DIAG == 2
                    if (rank == 0) mbar_arrive(&sm.full[s]);
#else
                    // both CTAs' loads complete on the leading CTA's barrier, which expects the bytes of both
                    const uint32_t bar = map_to_cta(smem_u32(&sm.full[s]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&sm.full[s], 2 * (1 + WIDE) * kXHalfBytes);
                    tma_load_4d_pair(sm.x[s], &map_x, bar, kb * kBlockK, t.row0 + int(rank) * kRowsPerHalf, 0, 0);
#pragma unroll
                    for (int h = 0; h < WIDE; ++h)
                        tma_load_4d_pair(sm.w[s] + h * kXHalfBytes, map_w, bar, kb * kBlockK,
                                         (t.hidden_tile * WIDE + h) * kHiddenPerTile, t.group, 0);
#endif
                }
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------------ leading CTA: tcgen05.mma issuer for the pair
        // The whole warp runs the loop (waits included) and one elected lane issues: see elect_one().
        {
            const bool elected = elect_one();
            constexpr uint32_t idesc = umma_idesc_bf16(2 * kRowsPerHalf, 2 * kHiddenPerTile, 0, 0);
            constexpr uint32_t desc_hi = umma_smem_desc_hi(1024);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++local) {
                // WIDE = 1: the two accumulators alternate; WIDE = 2: accumulator h belongs to hidden tile h of every tile
                const uint32_t a0 = WIDE == 1 ? (local & 1u) : 0u, use = WIDE == 1 ? (local >> 1) : local;
                if (use > 0) {                              // both CTAs' epilogues have read the accumulator(s)
#pragma unroll
                    for (uint32_t h = 0; h < uint32_t(WIDE); ++h)
                        ok = ok && mbar_wait_cluster(&sm.acc_empty[a0 + h], (use - 1u) & 1u, abort_flag, p.status, kGuAccEmpty);
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % kPairRing, use_s = it / kPairRing;
                    ok = mbar_wait(&sm.full[s], use_s & 1u, abort_flag, p.status, kGuFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t x_lo = umma_smem_desc_lo(smem_u32(sm.x[s]), 16);
                    const uint32_t w_lo = umma_smem_desc_lo(smem_u32(sm.w[s]), 16);
#if FPT_GATE_UP_DIAG != 3
#pragma unroll
                    for (uint32_t h = 0; h < uint32_t(WIDE); ++h) {
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / 16; ++k)
                            if (elected) umma_ss_words_pair(tmem + (a0 + h) * 256u, x_lo + 2u * k, w_lo + h * (kXHalfBytes / 16u) + 2u * k, desc_hi,
                                               idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
#endif
                    if (elected) umma_commit_pair(&sm.empty[s], 3);
                }
                if (ok) {
#pragma unroll
                    for (uint32_t h = 0; h < uint32_t(WIDE); ++h)
                        if (elected) umma_commit_pair(&sm.acc_full[a0 + h], 3);
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue (both CTAs, their own 128 rows)
        const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++local) {
            const Tile t = decode_tile<kRowsPerTile>(sm.table, p, tile);
            const uint32_t h = WIDE == 1 ? 0u : uint32_t(warp - 4) >> 2;       // which hidden tile of the row tile
            const uint32_t a = WIDE == 1 ? (local & 1u) : h, use = WIDE == 1 ? (local >> 1) : local;
            ok = mbar_wait(&sm.acc_full[a], use & 1u, abort_flag, p.status, kGuAccFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int row = t.row0 + int(rank) * kRowsPerHalf + 32 * (warp & 3) + lane;
            uint16_t* out_row = p.out + int64_t(row) * p.out_ld + (t.hidden_tile * WIDE + int(h)) * kHiddenPerTile;
            epilogue_rows(op, p, tmem + lane_base + a * 256u, out_row, row < t.row_end);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(&sm.acc_empty[a]);
                else mbar_arrive_cluster(map_to_cta(smem_u32(&sm.acc_empty[a]), 0));
            }
        }
    }
    // neither CTA may leave (or give back tensor memory) while the other can still reach its barriers or memory
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();
    if (warp == 2) tmem_dealloc_pair(tmem, kPairColumns);
}

// out = swish(gate) * up on packed bf16 lanes (the operator of fpt_swish_mul)
template <int SHAPE, int DEG>
struct PolySwishMul {
    ProgramWords p;
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<kBf16>::mul(eval_program<kBf16, SHAPE, DEG>(in[0], p), in[1]);
    }
};
struct NativeSwishMul {
    __device__ __forceinline__ void apply(const uint32_t (&in)[2], uint32_t (&out)[1]) const {
        out[0] = Pk<kBf16>::mul(eval_native<kBf16, kNatSwish>(in[0]), in[1]);
    }
};

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_gate_up_swiglu(void* out, const void* x, const void* w_gate, const void* w_up, int64_t rows, int64_t dim,
                                  int64_t hidden, int64_t x_ld, int64_t w_ld, int64_t w_group_stride, int64_t out_ld,
                                  const int32_t* group_ends, int64_t groups, int degree, int source, int epilogue,
                                  void* status, fpt_stream_t stream) {
    if (rows < 0 || dim <= 0 || hidden <= 0 || groups <= 0) return FPT_ERR_BAD_SIZE;
    if (groups > kMaxGroups || rows > 0x7fffffff - 2 * kRowsPerHalf || (groups > 1 && !group_ends)) return FPT_ERR_BAD_SIZE;
    if (hidden % kHiddenPerTile != 0 || dim % 8 != 0) return FPT_ERR_UNSUPPORTED_SHAPE;
    if (epilogue != FPT_GATE_UP_SWIGLU && epilogue != FPT_GATE_UP_RAW) return FPT_ERR_BAD_ENUM;
    if (source != FPT_SRC_CURRENT && source != FPT_SRC_SOLLYA) return FPT_ERR_BAD_ENUM;
    if (!status) return FPT_ERR_NULL_POINTER;
    if (rows == 0) return FPT_OK;
    if (!out || !x || !w_gate || !w_up) return FPT_ERR_NULL_POINTER;
    const int64_t out_width = epilogue == FPT_GATE_UP_RAW ? 2 * hidden : hidden;
    if (x_ld < dim || w_ld < dim || out_ld < out_width || w_group_stride < 0) return FPT_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(out) & 15u) || ((out_ld * 2) & 15)) return FPT_ERR_MISALIGNED;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;

    // 256-row tiles halve the weight bytes per row where the rows are plentiful and regular; ragged groups lose less of
    // a 128-row tile
    const int tile_rows_key = fpt::tuning_gate_up_tile_rows();
    // Measured (bench.py, extras.gate_up_swiglu_bf16.*.forms, three runs): in a loop long enough to meet the power cap pairs
    // of CTAs are 3 % (dense) to 7 % (grouped) ahead of the best single-CTA form; in isolated launches dense problems run
    // alike (1582 against 1590 TFLOP/s) and grouped ones 4 % faster on pairs.  An explicit tile height asks for the
    // single-CTA forms.
    const int pair_key = fpt::tuning_gate_up_cta_pair();
    const bool pair = pair_key == 1 || (pair_key < 0 && tile_rows_key == 0);
    const int halves = pair ? 2 : tile_rows_key ? tile_rows_key / kRowsPerHalf : (group_ends ? 1 : 2);
    const int tile_rows = halves * kRowsPerHalf;

    CUtensorMap map_x, map_wg, map_wu;
    {
        const uint64_t dims[4] = {uint64_t(dim), uint64_t(rows), 1, 1};
        const uint64_t strides[3] = {uint64_t(x_ld) * 2, uint64_t(x_ld) * 2 * uint64_t(rows), uint64_t(x_ld) * 2 * uint64_t(rows)};
        if (int rc = make_tensor_map_bf16_4d(&map_x, x, dims, strides, uint32_t(pair ? kRowsPerHalf : tile_rows))) return rc;
    }
    {
        const uint64_t group_bytes = groups > 1 ? uint64_t(w_group_stride) * 2 : uint64_t(w_ld) * 2 * uint64_t(hidden);
        const uint64_t dims[4] = {uint64_t(dim), uint64_t(hidden), uint64_t(groups), 1};
        const uint64_t strides[3] = {uint64_t(w_ld) * 2, group_bytes, group_bytes * uint64_t(groups)};
        if (int rc = make_tensor_map_bf16_4d(&map_wg, w_gate, dims, strides, kHiddenPerTile)) return rc;
        if (int rc = make_tensor_map_bf16_4d(&map_wu, w_up, dims, strides, kHiddenPerTile)) return rc;
    }
    GateUpParams p{};
    p.out = static_cast<uint16_t*>(out);
    p.group_ends = group_ends;
    p.out_ld = out_ld;
    p.rows = int(rows);
    p.hidden = int(hidden);
    p.groups = int(groups);
    p.hidden_tiles = int(hidden / kHiddenPerTile);
    p.k_blocks = int((dim + kBlockK - 1) / kBlockK);
    p.status = static_cast<uint32_t*>(status);

    static_assert(sizeof(GateUpSmem<1>) + 1024 <= 227 * 1024 && sizeof(GateUpSmem<2>) + 1024 <= 227 * 1024, "shared memory budget");
    // the number of tiles of a grouped problem is only known on the device: one CTA per SM, CTAs without a tile leave
    const int64_t dense_tiles = (rows + tile_rows - 1) / tile_rows * (hidden / kHiddenPerTile);
    const unsigned grid = unsigned(group_ends ? dev.sm_count : std::min<int64_t>(dense_tiles, dev.sm_count));
    auto launch_halves = [&](auto op, auto halves_c) {
        constexpr int H = decltype(halves_c)::value;
        const size_t smem = sizeof(GateUpSmem<H>) + 1024;
        auto kernel = gate_up_swiglu_kernel<decltype(op), H>;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
        kernel<<<grid, 128 + 128 * H, smem, stream>>>(map_x, map_wg, map_wu, p, op);
        return cuda_status(cudaGetLastError());
    };
    // two hidden tiles per row tile of a pair where asked for (tuning key gate_up_pair_wide) and their number is even
    const bool wide = pair && (hidden / kHiddenPerTile) % 2 == 0 && fpt::tuning_gate_up_pair_wide() != 0;
    auto launch_pair_wide = [&](auto op, auto wide_c) {
        constexpr int W = decltype(wide_c)::value;
        GateUpParams pw = p;
        pw.hidden_tiles = p.hidden_tiles / W;               // the table counts tiles of W hidden tiles
        const size_t smem = sizeof(GateUpPairSmem<W>) + 1024;
        static_assert(sizeof(GateUpPairSmem<W>) + 1024 <= 227 * 1024, "shared memory budget");
        auto kernel = gate_up_swiglu_pair_kernel<decltype(op), W>;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
        const int64_t tiles = (rows + 2 * kRowsPerHalf - 1) / (2 * kRowsPerHalf) * pw.hidden_tiles;
        const int64_t pairs = std::min<int64_t>(group_ends ? dev.sm_count / 2 : tiles, dev.sm_count / 2);
        kernel<<<unsigned(2 * pairs), 128 + 128 * W, smem, stream>>>(map_x, map_wg, map_wu, pw, op);   // clusters of two (kernel attribute)
        return cuda_status(cudaGetLastError());
    };
    auto launch_pair = [&](auto op) { return wide ? launch_pair_wide(op, IC<2>{}) : launch_pair_wide(op, IC<1>{}); };
    auto launch = [&](auto op) {
        if (pair) return launch_pair(op);
        return halves == 2 ? launch_halves(op, IC<2>{}) : launch_halves(op, IC<1>{});
    };
    if (epilogue == FPT_GATE_UP_RAW) return launch(RawEpilogue{});
    if (degree == 0) return launch(NativeSwishMul{});
    const ProgramRow* row = find_program(FPT_FN_SWISH, FPT_FWD, degree, FPT_BF16, source);
    if (!row || row->degree != 3) return FPT_ERR_UNKNOWN_PROGRAM;      // the B1 / B4 program is the cubic
    const ProgramWords words = program_words(*row);
    if (row->shape == kSwish) return launch(PolySwishMul<kSwish, 3>{words});
    if (row->shape == kXmulHalf) return launch(PolySwishMul<kXmulHalf, 3>{words});
    return FPT_ERR_UNSUPPORTED_SHAPE;
}
