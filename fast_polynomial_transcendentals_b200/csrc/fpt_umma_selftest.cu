// Self-test of the two tensor-core building blocks of the attention kernel on one 128x128x128 tile:
//   mode 0:  C = A * B^T   both operands K-major in shared memory (the Q K^T form)
//   mode 1:  C = P * V     P (bf16) staged in tensor memory, V as an MN-major shared-memory operand (the P V form)
//   mode 2:  C = A^T * B   A written to shared memory by the threads themselves in the swizzled panel layout and read as
//                          an MN-major A operand, B MN-major (the dQ += dS K form of the fused attention backward)
// It exists so that descriptor encodings are validated against a plain matrix product before the full pipeline
// depends on them, and it stays in the library as a diagnostic entry point.
#include <cstring>

#include "fpt_common.h"
#include "fpt_sm100.cuh"

namespace fpt {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}
}  // namespace

int make_tensor_map_bf16_4d(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                            uint32_t box_rows) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return FPT_ERR_NO_DEVICE;
    if (reinterpret_cast<uintptr_t>(base) & 15u) return FPT_ERR_MISALIGNED;
    for (int i = 0; i < 3; ++i)
        if (strides_bytes[i] & 15u) return FPT_ERR_MISALIGNED;
    cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t gstride[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
    cuuint32_t box[4] = {64u, box_rows, 1u, 1u};
    cuuint32_t estride[4] = {1u, 1u, 1u, 1u};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstride, box, estride,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FPT_OK : FPT_ERR_BAD_SIZE;
}

namespace {

using namespace sm100;

constexpr int kTile = 128;
constexpr uint32_t kPanelBytes = kTile * 128;  // 128 rows x 128 bytes

struct SelftestSmem {
    alignas(1024) uint8_t a[2 * kPanelBytes];
    alignas(1024) uint8_t b[2 * kPanelBytes];
    alignas(8) uint64_t bar_load;
    uint64_t bar_mma;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __grid_constant__ CUtensorMap map_a,
                                                            const __grid_constant__ CUtensorMap map_b,
                                                            const uint16_t* __restrict__ p_global, float* __restrict__ c,
                                                            int mode, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    SelftestSmem& s = *reinterpret_cast<SelftestSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&s.bar_load, 1);
        mbar_init(&s.bar_mma, 1);
        s.abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(&s.tmem_base, 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s.tmem_base;
    const uint32_t tmem_c = tmem;        // 128 fp32 columns
    const uint32_t tmem_p = tmem + 128;  // 64 columns of packed bf16
    volatile uint32_t* abort_flag = &s.abort_flag;

    if (mode == 1) {  // stage P: thread t owns row t; 128 bf16 = 64 words
        uint32_t words[32];
        const uint32_t lane_addr = tmem_p + (uint32_t(warp * 32) << 16);
        const uint32_t* row = reinterpret_cast<const uint32_t*>(p_global) + size_t(threadIdx.x) * 64;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int i = 0; i < 32; ++i) words[i] = row[half * 32 + i];
            tmem_st_32x32b_x32(lane_addr + half * 32, words);
        }
        tmem_st_wait();
        tc_fence_before_sync();
    }
    if (mode == 2) {  // thread t owns row t (a K index) of A: 128 bf16 = two panels of eight 16-byte chunks, chunk c of
                      // row t stored at chunk position c ^ (t % 8) of its 128-byte line (the 128-byte swizzle TMA applies)
        const uint4* row = reinterpret_cast<const uint4*>(p_global + size_t(threadIdx.x) * 128);
#pragma unroll
        for (int panel = 0; panel < 2; ++panel)
#pragma unroll
            for (int chunk = 0; chunk < 8; ++chunk)
                *reinterpret_cast<uint4*>(s.a + panel * kPanelBytes + threadIdx.x * 128 + ((chunk ^ (threadIdx.x & 7)) << 4)) =
                    row[panel * 8 + chunk];
        fence_async_shared();     // generic-proxy stores, read next by the tensor core through the async proxy
    }
    __syncthreads();
    tc_fence_after_sync();

    if (threadIdx.x == 0) {
        const uint32_t bytes = (mode == 0 ? 4u : 2u) * kPanelBytes;
        mbar_arrive_expect_tx(&s.bar_load, bytes);
        if (mode == 0) {
            tma_load_4d(s.a, &map_a, &s.bar_load, 0, 0, 0, 0);
            tma_load_4d(s.a + kPanelBytes, &map_a, &s.bar_load, 64, 0, 0, 0);
        }
        tma_load_4d(s.b, &map_b, &s.bar_load, 0, 0, 0, 0);
        tma_load_4d(s.b + kPanelBytes, &map_b, &s.bar_load, 64, 0, 0, 0);
        if (mbar_wait(&s.bar_load, 0, abort_flag, status, 1)) {
            tc_fence_after_sync();
            if (mode == 0) {
                constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t off = uint32_t(k >> 2) * kPanelBytes + uint32_t(k & 3) * 32u;
                    umma_ss(tmem_c, umma_smem_desc(smem_u32(s.a) + off, 16, 1024), umma_smem_desc(smem_u32(s.b) + off, 16, 1024),
                            idesc, k > 0);
                }
            } else if (mode == 2) {
                constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 1, 1);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_ss(tmem_c, umma_smem_desc(smem_u32(s.a) + uint32_t(k) * 2048u, kPanelBytes, 1024),
                            umma_smem_desc(smem_u32(s.b) + uint32_t(k) * 2048u, kPanelBytes, 1024), idesc, k > 0);
            } else {
                constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 1);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_ts(tmem_c, tmem_p + 8u * k, umma_smem_desc(smem_u32(s.b) + uint32_t(k) * 2048u, kPanelBytes, 1024), idesc,
                            k > 0);
            }
            umma_commit(&s.bar_mma);
        }
    }
    const bool ok = mbar_wait(&s.bar_mma, 0, abort_flag, status, 2);
    tc_fence_after_sync();
    if (ok) {
        const uint32_t lane_addr = tmem_c + (uint32_t(warp * 32) << 16);
        float* out = c + size_t(threadIdx.x) * 128;
#pragma unroll
        for (int chunk = 0; chunk < 4; ++chunk) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(lane_addr + chunk * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) out[chunk * 32 + i] = __uint_as_float(v[i]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// The bounded wait of the attention kernels on a barrier nobody arrives on: one thread, one mbarrier, no TMA, no tensor
// memory, no tensor-core operation, so the block that gives up has nothing in flight.  report[0]: 1 = the wait ran out,
// 2 = the block found the status word already set and did not wait, 3 = the wait succeeded (cannot happen);
// report[1], report[2]: low / high word of the nanoseconds spent waiting.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(uint32_t* status, uint32_t* report, uint64_t limit_ns,
                                                                   uint32_t where) {
    __shared__ alignas(8) uint64_t bar;
    __shared__ uint32_t abort_word;
    if (threadIdx.x != 0) return;
    volatile uint32_t* abort_flag = &abort_word;
    mbar_init(&bar, 1);
    abort_word = *reinterpret_cast<volatile uint32_t*>(status) != 0u ? 1u : 0u;   // the attention kernels' entry check
    mbar_fence_init();
    if (*abort_flag) {
        report[0] = 2u;
        report[1] = report[2] = 0u;
        return;
    }
    const uint64_t t0 = global_timer_ns();
    const bool ok = mbar_wait(&bar, 0, abort_flag, status, where, limit_ns);
    const uint64_t dt = global_timer_ns() - t0;
    report[0] = ok ? 3u : 1u;
    report[1] = uint32_t(dt);
    report[2] = uint32_t(dt >> 32);
}

}  // namespace
}  // namespace fpt

using namespace fpt;

extern "C" int fpt_selftest_bounded_wait(void* status, void* report, int64_t limit_ns, int where, fpt_stream_t stream) {
    if (!status || !report) return FPT_ERR_NULL_POINTER;
    if (limit_ns < 1000 || limit_ns > 1000000) return FPT_ERR_BAD_SIZE;     // 1 us .. 1 ms
    if (where < 1 || where > 0xffff) return FPT_ERR_BAD_ENUM;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(static_cast<uint32_t*>(status), static_cast<uint32_t*>(report),
                                                       uint64_t(limit_ns), uint32_t(where));
    return cuda_status(cudaGetLastError());
}

// a, b: bf16 [128, 128] row-major device arrays; c: fp32 [128, 128]; status: one device word, 0 on success.
// mode 0: c = a * b^T.  mode 1: c = a * b.  mode 2: c = a^T * b.
extern "C" int fpt_selftest_umma(void* c, const void* a, const void* b, int mode, void* status, fpt_stream_t stream) {
    if (!c || !a || !b || !status) return FPT_ERR_NULL_POINTER;
    if (mode < 0 || mode > 2) return FPT_ERR_BAD_ENUM;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev)) return rc;
    const uint64_t dims[4] = {128, 128, 1, 1};
    const uint64_t strides[3] = {256, 256 * 128, 256 * 128};
    CUtensorMap map_a, map_b;
    if (int rc = make_tensor_map_bf16_4d(&map_a, a, dims, strides, 128)) return rc;
    if (int rc = make_tensor_map_bf16_4d(&map_b, b, dims, strides, 128)) return rc;
    const size_t smem = sizeof(SelftestSmem) + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    umma_selftest_kernel<<<1, 128, smem, stream>>>(map_a, map_b, static_cast<const uint16_t*>(a), static_cast<float*>(c), mode,
                                                   static_cast<uint32_t*>(status));
    return cuda_status(cudaGetLastError());
}
