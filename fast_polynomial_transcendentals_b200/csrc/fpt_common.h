// Host-side helpers shared by every translation unit of the library: status codes,
// per-device facts (queried once per device, never assumed from device 0) and the few
// launch knobs that benchmarks may override.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/fpt_b200.h"

namespace fpt {

struct DeviceInfo {
    int device;
    int sm_count;
    int64_t l2_bytes;
    int cc_major, cc_minor;
};

struct Tuning {
    int blocks_per_sm;  // persistent-grid cap: blocks per SM (0 = one block per tile, no cap)
    int streaming;      // -1 decide from footprint vs L2, 0 never, 1 always
};

int current_device_info(DeviceInfo* out);
Tuning tuning();
// attention kernels, order in which blocks are handed out: 0 heads fastest, 1 row blocks of one head fastest,
// -1 (default) picks by the size of the K/V working set of the blocks that run together
int tuning_attention_raster();
int tuning_attention_bwd_fused();
int tuning_gate_up_pair_wide();     // pairs of CTAs: 1 two hidden tiles per row tile where their number is even, 0 (default) one
int tuning_gate_up_cta_pair();      // gate / up projection on pairs of CTAs (cta_group::2): 1 always, 0 never, -1 (default) unless a tile height is named
int tuning_attention_cta_pair();    // attention forward on pairs of CTAs (cta_group::2) where two blocks share their K / V: 0 never, 1 where possible
int tuning_gate_up_tile_rows();     // gate / up projection: rows per tile, 128 or 256 (0: 256 for dense, 128 for grouped problems)
int tuning_rope_heads_per_block();   // fused RoPE: heads one block rotates (0: all of them)
int tuning_attention_split();    // attention forward, column-split score-mod warps: 0 never, 1 soft-capped mode (default), 2 sigmoid mode too

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? FPT_OK : int(e); }

}  // namespace fpt
