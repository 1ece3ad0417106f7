// Microbenchmark (not part of the library; build and run by hand on a B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o reduce_add_rate reduce_add_rate.cu && ./reduce_add_rate
// fp32 reduce-add throughput of one SM into global memory: the copy engine (cp.reduce.async.bulk ... add.f32) by copy size
// and copies in flight, into a destination that stays in L2 or not, and red.global.add.f32 from four warps.  The figures
// it printed are in the profile notes of the attention backward.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
template <int INFLIGHT>
__global__ void __launch_bounds__(128, 1) bulk_kernel(float* dst, size_t region_floats, int chunk_bytes, int iters, int shared_dst) {
    extern __shared__ __align__(1024) uint8_t smem[];
    for (int i = threadIdx.x; i < 4 * chunk_bytes / 4; i += blockDim.x) reinterpret_cast<float*>(smem)[i] = 1.0f;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    float* base = dst + (shared_dst ? 0 : size_t(blockIdx.x) * region_floats);
    const size_t chunk_floats = chunk_bytes / 4;
    const size_t slots = region_floats / chunk_floats;
    if (threadIdx.x == 0) {
        for (int i = 0; i < iters; ++i) {
            size_t slot = (size_t(i) * (shared_dst ? 7 : 1) + (shared_dst ? blockIdx.x * 13 : 0)) % slots;
            asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                         :: "l"(base + slot * chunk_floats), "r"(smem_u32(smem + (i % 4) * chunk_bytes)), "r"(chunk_bytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(INFLIGHT - 1) : "memory");
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}
__global__ void __launch_bounds__(128, 1) red_kernel(float* dst, size_t region_floats, int iters) {
    float* base = dst + size_t(blockIdx.x) * region_floats;
    const size_t lines = region_floats / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = 0; i < iters; ++i) {
        size_t line = (size_t(i) * 4 + warp) % lines;
        asm volatile("red.global.add.f32 [%0], %1;" :: "l"(base + line * 32 + lane), "f"(1.0f) : "memory");
    }
}
int main() {
    int sms = 0; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    int clk = 0; cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, 0);
    const size_t total = size_t(sms) * (8u << 20);             // 8 MiB per CTA: 1.2 GB, beyond L2
    float* dst; cudaMalloc(&dst, total); cudaMemset(dst, 0, total);
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    auto run = [&](const char* name, auto launch, double bytes) {
        launch(); cudaDeviceSynchronize();
        cudaEventRecord(a); launch(); cudaEventRecord(b); cudaEventSynchronize(b);
        float ms; cudaEventElapsedTime(&ms, a, b);
        cudaError_t e = cudaGetLastError();
        printf("%-64s %8.3f ms  %7.1f GB/s total  %6.2f GB/s per SM  (%s)\n", name, ms, bytes / ms / 1e6, bytes / ms / 1e6 / sms, cudaGetErrorString(e));
    };
    const int chunks[] = {4096, 16384, 32768};
    for (int region_kb : {64, 8192}) {                          // per-CTA destination region: L2-resident or not
        for (int cb : chunks) {
            const int iters = (64 << 20) / cb;                  // 64 MiB per CTA
            const size_t rf = size_t(region_kb) * 1024 / 4;
            char name[128];
            auto go = [&](auto kern, int inflight) {
                cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * cb);
                snprintf(name, sizeof name, "bulk reduce %5d B, %d in flight, region %5d KiB per CTA", cb, inflight, region_kb);
                run(name, [&] { kern<<<sms, 128, 4 * cb>>>(dst, rf, cb, iters, 0); }, double(sms) * iters * cb);
            };
            go(bulk_kernel<1>, 1); go(bulk_kernel<2>, 2); go(bulk_kernel<4>, 4);
        }
        char name[128];
        snprintf(name, sizeof name, "red.global.add.f32, 4 warps x 128 B, region %5d KiB per CTA", region_kb);
        const int iters = 1 << 17;
        run(name, [&] { red_kernel<<<sms, 128>>>(dst, size_t(region_kb) * 1024 / 4, iters); }, double(sms) * iters * 512);
    }
    {   // all CTAs add into one shared 32 MiB region (several CTAs per line over time, like the dQ buffer)
        const int cb = 16384, iters = (64 << 20) / cb;
        cudaFuncSetAttribute(bulk_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * cb);
        run("bulk reduce 16384 B, 3 in flight, one shared 32 MiB region", [&] { bulk_kernel<3><<<sms, 128, 4 * cb>>>(dst, (32u << 20) / 4, cb, iters, 1); }, double(sms) * iters * cb);
    }
    printf("sms %d clock %d kHz\n", sms, clk);
    return 0;
}
