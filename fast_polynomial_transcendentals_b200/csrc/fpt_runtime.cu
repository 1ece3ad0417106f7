// Process-wide host state: per-device facts, launch knobs, the program table and status strings.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "fpt_programs.h"

namespace fpt {

namespace {
constexpr int kMaxDevices = 64;
struct DeviceSlot {
    std::atomic<int> ready{0};
    DeviceInfo info{};
};
DeviceSlot g_devices[kMaxDevices];
std::mutex g_device_mutex;
std::atomic<int> g_blocks_per_sm{0};
std::atomic<int> g_streaming{-1};
std::atomic<int> g_attention_split{1};
std::atomic<int> g_attention_raster{-1};
std::atomic<int> g_attention_bwd_fused{1};
std::atomic<int> g_gate_up_tile_rows{0};
std::atomic<int> g_attention_cta_pair{0};
std::atomic<int> g_gate_up_cta_pair{-1};
std::atomic<int> g_gate_up_pair_wide{0};
std::atomic<int> g_rope_heads_per_block{8};   // measured: 8 is 1.5-3 % ahead of "all heads in one block" at 32 heads

enum { DT_FP16 = kFp16, DT_BF16 = kBf16 };
enum { SRC_CURRENT = FPT_SRC_CURRENT, SRC_SOLLYA = FPT_SRC_SOLLYA };
enum { SH_ODD_HALF = kOddHalf, SH_ODD = kOdd, SH_ODD_SAT = kOddSat, SH_SWISH = kSwish, SH_XMUL_HALF = kXmulHalf,
       SH_EVEN = kEven, SH_ALG_SIG = kAlgSig, SH_ALG_TANH = kAlgTanh };
#define FPT_PROGRAM(NAME, DT, SRC, SHAPE, DEG, CLAMP, C0, C1, C2, C3, C4, C5, C6) \
    { #NAME, DT_##DT, SRC_##SRC, SH_##SHAPE, DEG, CLAMP, { C0, C1, C2, C3, C4, C5, C6 } },
const ProgramRow k_rows[] = {
#include "fpt_program_table.inc"
};
#undef FPT_PROGRAM
constexpr int k_row_count = int(sizeof(k_rows) / sizeof(k_rows[0]));
}  // namespace

int current_device_info(DeviceInfo* out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ? FPT_ERR_NO_DEVICE : int(e);
    if (device < 0 || device >= kMaxDevices) return FPT_ERR_NO_DEVICE;
    DeviceSlot& slot = g_devices[device];
    if (!slot.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_device_mutex);
        if (!slot.ready.load(std::memory_order_relaxed)) {
            DeviceInfo info{};
            info.device = device;
            int l2 = 0;
            if ((e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return int(e);
            if ((e = cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, device)) != cudaSuccess) return int(e);
            if ((e = cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, device)) != cudaSuccess) return int(e);
            if ((e = cudaDeviceGetAttribute(&info.cc_minor, cudaDevAttrComputeCapabilityMinor, device)) != cudaSuccess) return int(e);
            info.l2_bytes = l2;
            slot.info = info;
            slot.ready.store(1, std::memory_order_release);
        }
    }
    *out = slot.info;
    if (out->cc_major != 10) return FPT_ERR_NO_DEVICE;
    return FPT_OK;
}

Tuning tuning() { return Tuning{g_blocks_per_sm.load(), g_streaming.load()}; }
int tuning_attention_split() { return g_attention_split.load(); }
int tuning_attention_raster() { return g_attention_raster.load(); }
int tuning_attention_bwd_fused() { return g_attention_bwd_fused.load(); }
int tuning_gate_up_tile_rows() { return g_gate_up_tile_rows.load(); }
int tuning_attention_cta_pair() { return g_attention_cta_pair.load(); }
int tuning_gate_up_cta_pair() { return g_gate_up_cta_pair.load(); }
int tuning_gate_up_pair_wide() { return g_gate_up_pair_wide.load(); }
int tuning_rope_heads_per_block() { return g_rope_heads_per_block.load(); }

const ProgramRow* program_table(int* count) {
    if (count) *count = k_row_count;
    return k_rows;
}

namespace {
// [function][direction][degree-3][dtype][source] -> row index + 1 (0 = none), filled once.
struct ProgramIndex {
    unsigned char slot[5][2][4][2][2];
    ProgramIndex() {
        static const char* const fn_names[] = {"SIGMOID", "TANH", "SWISH", "ERF", "GELU"};
        std::memset(slot, 0, sizeof(slot));
        for (int i = 0; i < k_row_count; ++i) {
            const ProgramRow& r = k_rows[i];
            for (int f = 0; f < 5; ++f)
                for (int d = 0; d < 2; ++d) {
                    char name[32];
                    std::snprintf(name, sizeof(name), "%s_%s_D%d", fn_names[f], d == 0 ? "FWD" : "BWD", r.degree);
                    if (r.degree >= 3 && r.degree <= 6 && !std::strcmp(r.name, name))
                        slot[f][d][r.degree - 3][r.dtype][r.source] = (unsigned char)(i + 1);
                }
        }
    }
};
}  // namespace

const ProgramRow* find_program(int function, int direction, int degree, int dtype, int source) {
    static const ProgramIndex index;
    if (function < 0 || function > FPT_FN_GELU || (direction != FPT_FWD && direction != FPT_BWD)) return nullptr;
    if (degree < 3 || degree > 6 || dtype < 0 || dtype > 1 || source < 0 || source > 1) return nullptr;
    const int s = index.slot[function][direction][degree - 3][dtype][source];
    return s ? &k_rows[s - 1] : nullptr;
}

}  // namespace fpt

extern "C" {

const char* fpt_status_string(int status) {
    switch (status) {
    case FPT_OK: return "ok";
    case FPT_ERR_NULL_POINTER: return "null pointer argument";
    case FPT_ERR_BAD_SIZE: return "size argument out of range";
    case FPT_ERR_MISALIGNED: return "pointer is not aligned as required";
    case FPT_ERR_UNKNOWN_PROGRAM: return "no polynomial program for this function/direction/degree/dtype/source";
    case FPT_ERR_BAD_ENUM: return "enumeration argument out of range";
    case FPT_ERR_UNSUPPORTED_SHAPE: return "operation not defined for this program shape";
    case FPT_ERR_NO_DEVICE: return "no usable CUDA device of compute capability 10.x is current";
    case FPT_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case FPT_ERR_SCRATCH_TOO_SMALL: return "the problem needs more scratch than the library's fixed array holds";
    default: return status > 0 ? cudaGetErrorString(cudaError_t(status)) : "unknown status";
    }
}

const char* fpt_version(void) { return "fpt_b200 0.1 sm_100a"; }

int fpt_program_count(void) { return fpt::k_row_count; }

int fpt_program_info(int index, char* name_out, int name_capacity, int* dtype, int* source, int* shape, int* degree,
                     uint16_t* clamp, uint16_t* coeffs7) {
    if (index < 0 || index >= fpt::k_row_count) return FPT_ERR_BAD_SIZE;
    const fpt::ProgramRow& r = fpt::k_rows[index];
    if (name_out && name_capacity > 0) {
        std::strncpy(name_out, r.name, size_t(name_capacity) - 1);
        name_out[name_capacity - 1] = 0;
    }
    if (dtype) *dtype = r.dtype;
    if (source) *source = r.source;
    if (shape) *shape = r.shape;
    if (degree) *degree = r.degree;
    if (clamp) *clamp = r.clamp;
    if (coeffs7) std::memcpy(coeffs7, r.c, sizeof(r.c));
    return FPT_OK;
}

int fpt_set_tuning(const char* key, int value) {
    if (!key) return FPT_ERR_NULL_POINTER;
    if (!std::strcmp(key, "blocks_per_sm")) { if (value < 0 || value > 64) return FPT_ERR_BAD_SIZE; fpt::g_blocks_per_sm = value; return FPT_OK; }
    if (!std::strcmp(key, "streaming")) { if (value < -1 || value > 1) return FPT_ERR_BAD_SIZE; fpt::g_streaming = value; return FPT_OK; }
    if (!std::strcmp(key, "attention_split")) { if (value < 0 || value > 2) return FPT_ERR_BAD_SIZE; fpt::g_attention_split = value; return FPT_OK; }
    if (!std::strcmp(key, "attention_raster")) { if (value < -1 || value > 1) return FPT_ERR_BAD_SIZE; fpt::g_attention_raster = value; return FPT_OK; }
    if (!std::strcmp(key, "attention_bwd_fused")) { if (value < 0 || value > 2) return FPT_ERR_BAD_SIZE; fpt::g_attention_bwd_fused = value; return FPT_OK; }
    if (!std::strcmp(key, "rope_heads_per_block")) { if (value < 0 || value > 65535) return FPT_ERR_BAD_SIZE; fpt::g_rope_heads_per_block = value; return FPT_OK; }
    if (!std::strcmp(key, "gate_up_tile_rows")) { if (value != 0 && value != 128 && value != 256) return FPT_ERR_BAD_SIZE; fpt::g_gate_up_tile_rows = value; return FPT_OK; }
    if (!std::strcmp(key, "attention_cta_pair")) { if (value < 0 || value > 1) return FPT_ERR_BAD_SIZE; fpt::g_attention_cta_pair = value; return FPT_OK; }
    if (!std::strcmp(key, "gate_up_pair_wide")) { if (value < 0 || value > 1) return FPT_ERR_BAD_SIZE; fpt::g_gate_up_pair_wide = value; return FPT_OK; }
    if (!std::strcmp(key, "gate_up_cta_pair")) { if (value < -1 || value > 1) return FPT_ERR_BAD_SIZE; fpt::g_gate_up_cta_pair = value; return FPT_OK; }
    return FPT_ERR_BAD_ENUM;
}

int fpt_get_tuning(const char* key, int* value) {
    if (!key || !value) return FPT_ERR_NULL_POINTER;
    if (!std::strcmp(key, "blocks_per_sm")) { *value = fpt::g_blocks_per_sm; return FPT_OK; }
    if (!std::strcmp(key, "streaming")) { *value = fpt::g_streaming; return FPT_OK; }
    if (!std::strcmp(key, "attention_split")) { *value = fpt::g_attention_split; return FPT_OK; }
    if (!std::strcmp(key, "attention_raster")) { *value = fpt::g_attention_raster; return FPT_OK; }
    if (!std::strcmp(key, "attention_bwd_fused")) { *value = fpt::g_attention_bwd_fused; return FPT_OK; }
    if (!std::strcmp(key, "rope_heads_per_block")) { *value = fpt::g_rope_heads_per_block; return FPT_OK; }
    if (!std::strcmp(key, "gate_up_tile_rows")) { *value = fpt::g_gate_up_tile_rows; return FPT_OK; }
    if (!std::strcmp(key, "attention_cta_pair")) { *value = fpt::g_attention_cta_pair; return FPT_OK; }
    if (!std::strcmp(key, "gate_up_pair_wide")) { *value = fpt::g_gate_up_pair_wide; return FPT_OK; }
    if (!std::strcmp(key, "gate_up_cta_pair")) { *value = fpt::g_gate_up_cta_pair; return FPT_OK; }
    return FPT_ERR_BAD_ENUM;
}

}  // extern "C"
