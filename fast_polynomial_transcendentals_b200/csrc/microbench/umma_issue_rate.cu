// Microbenchmark (not part of the library; build and run by hand on a B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 --expt-relaxed-constexpr -o umma_issue_rate umma_issue_rate.cu -lcuda
//   ./umma_issue_rate
// Cycles per tcgen05.mma (kind::f16, bf16, M = 128, K = 16) by N, operand source and operand layout: one block per SM, a
// long stream of products over the same shared-memory tiles, issued either by one lane inside a branch or by a converged
// warp with an elected lane, alone or next to background work of the kinds the attention kernels have (tensor-memory loads
// and stores, shared-memory stores, bulk loads, one warp of dependent FMAs per scheduler).  Also the exact product
// sequence of one half step of the single-pass attention backward.  Every wait is bounded.  The figures it printed are in
// the profile notes of the attention kernels; they are why the issuing warps of the library run converged.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../fpt_sm100.cuh"
using namespace fpt::sm100;
struct Smem {
    alignas(1024) uint8_t a[32768];
    alignas(1024) uint8_t b[32768];
    alignas(8) uint64_t done;
    uint64_t sink;
    uint64_t ld_bar;
    uint32_t tmem_base;
    uint32_t stop;
    alignas(1024) uint8_t scratch[32768];
};
// variant: 0 SS K-major/K-major, 1 SS MN/MN, 2 TS with B MN-major, 3 TS with B K-major
template <int N, int VARIANT, int BG>
__global__ void __launch_bounds__(256, 1) mma_kernel(unsigned long long* cycles, int rounds, const uint8_t* src) {
    extern __shared__ uint8_t raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 65536 / 4; i += 256) reinterpret_cast<uint32_t*>(sm.a)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) { mbar_init(&sm.done, 1); mbar_init(&sm.sink, 1000000); mbar_init(&sm.ld_bar, 1); mbar_fence_init(); sm.stop = 0; }
    fence_async_shared();
    if (warp == 0) { tmem_alloc(&sm.tmem_base, 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const bool converged = (BG & 128) != 0;
    uint32_t elected = 1;
    if (converged && warp == 1) asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    if (converged ? warp == 1 : threadIdx.x == 32) {
        constexpr uint32_t desc_hi = umma_smem_desc_hi(1024);
        constexpr uint32_t idesc = umma_idesc_bf16(128, N, VARIANT == 1 ? 1 : 0, (VARIANT == 1 || VARIANT == 2) ? 1 : 0);
        const uint32_t a_k = umma_smem_desc_lo(smem_u32(sm.a), 16), b_k = umma_smem_desc_lo(smem_u32(sm.b), 16);
        const uint32_t a_mn = umma_smem_desc_lo(smem_u32(sm.a), 16384), b_mn = umma_smem_desc_lo(smem_u32(sm.b), N == 64 && VARIANT != 1 ? 8192 : 16384);
        const long long t0 = clock64();
        if (VARIANT >= 9) {
            // the half-step sequence of the pipelined attention backward: dK (4 TS N=128), dV (4 TS N=128), dQ^T (8 SS MN/MN
            // N=64), commit x2, dP^T (8 SS K/K N=64), S^T (8 SS K/K N=64), commit.  VARIANT 10: everything N=128-equivalent
            // work as N=128 products (4 + 4 + 4 + 4 + 4), for comparison.
            constexpr uint32_t id_ts = umma_idesc_bf16(128, 128, 0, 1);
            constexpr uint32_t id_mnmn64 = umma_idesc_bf16(128, 64, 1, 1);
            constexpr uint32_t id_kk64 = umma_idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t id_mnmn128 = umma_idesc_bf16(128, 128, 1, 1);
            constexpr uint32_t id_kk128 = umma_idesc_bf16(128, 128, 0, 0);
            for (int r = 0; r < rounds; ++r) {
                const uint32_t hh = uint32_t(r & 1) * 64u;
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_ts_words(tmem + 256u, tmem + 128u + hh + 32u * (k >> 1) + 8u * (k & 1), b_mn + uint32_t(k) * 128u, desc_hi, id_ts, 1);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_ts_words(tmem + 384u, tmem + 128u + hh + 32u * (k >> 1) + 16u + 8u * (k & 1), b_mn + uint32_t(k) * 128u, desc_hi, id_ts, 1);
                if (VARIANT == 9) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) umma_ss_words(tmem + hh, a_mn + uint32_t(kk) * 128u, b_mn + uint32_t(kk) * 128u, desc_hi, id_mnmn64, kk > 0);
                } else {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) umma_ss_words(tmem, a_mn + uint32_t(kk) * 128u, b_mn + uint32_t(kk) * 128u, desc_hi, id_mnmn128, kk > 0);
                }
                umma_commit(&sm.sink);
                umma_commit(&sm.sink);
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {
                    if (VARIANT == 9) {
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const uint32_t off_k = (uint32_t(kk >> 2) * 16384u + uint32_t(kk & 3) * 32u) / 16u;
                            umma_ss_words(tmem + (pass == 0 ? 128u : 0u) + hh, a_k + off_k, b_k + off_k, desc_hi, id_kk64, kk > 0);
                        }
                    } else {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint32_t off_k = (uint32_t(kk >> 2) * 16384u + uint32_t(kk & 3) * 32u) / 16u;
                            umma_ss_words(tmem + (pass == 0 ? 128u : 0u), a_k + off_k, b_k + off_k, desc_hi, id_kk128, kk > 0);
                        }
                    }
                }
                umma_commit(&sm.sink);
            }
        } else
        for (int r = 0; r < rounds; ++r) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t off_k = (uint32_t(kk >> 2) * 16384u + uint32_t(kk & 3) * 32u) / 16u;
                const uint32_t off_mn = uint32_t(kk) * (2048u / 16u);
                const uint32_t d = tmem + 256u * uint32_t(r & 1);     // two accumulators alternate
                const uint32_t accum = (BG & 16) ? (kk > 0) : 1;
                if (VARIANT == 0) { if (elected) umma_ss_words(d, a_k + off_k, b_k + off_k, desc_hi, idesc, accum); }
                else if (VARIANT == 1) umma_ss_words(d, a_mn + off_mn, b_mn + off_mn, desc_hi, idesc, 1);
                else if (VARIANT == 2) umma_ts_words(d, tmem + 128u + 8u * uint32_t(kk), b_mn + off_mn, desc_hi, idesc, 1);
                else umma_ts_words(d, tmem + 128u + 8u * uint32_t(kk), b_k + off_k, desc_hi, idesc, 1);
            }
            if (BG & 8) umma_commit(&sm.sink);
        }
        if (elected) umma_commit(&sm.done);
        if (converged) __syncwarp();
        uint32_t spins = 0;
        while (!mbar_try_wait(&sm.done, 0) && ++spins < (1u << 28)) { }
        const long long t1 = clock64();
        if (elected) cycles[blockIdx.x] = (unsigned long long)(t1 - t0);
        *reinterpret_cast<volatile uint32_t*>(&sm.stop) = 1u;
    } else if (warp == 4 && (BG & 32) != 0) {
        // background bulk loads global -> shared, 32 KiB per round, one thread
        if ((threadIdx.x & 31) == 0) {
            for (int it = 0; it < (1 << 20); ++it) {
                mbar_arrive_expect_tx(&sm.ld_bar, 32768);
                bulk_load_1d(sm.scratch, src + size_t((it * 2 + blockIdx.x * 7) & 31) * 32768, 16384, &sm.ld_bar);
                bulk_load_1d(sm.scratch + 16384, src + size_t((it * 2 + 1 + blockIdx.x * 7) & 31) * 32768, 16384, &sm.ld_bar);
                uint32_t spins = 0;
                while (!mbar_try_wait(&sm.ld_bar, uint32_t(it) & 1u) && ++spins < (1u << 24)) { }
                if (*reinterpret_cast<volatile uint32_t*>(&sm.stop)) break;
            }
        }
    } else if (warp >= 4 && (BG & 64) != 0) {
        // background arithmetic on every scheduler (warps 4..7 = one per scheduler; warp 5 shares the issuer's)
        float a0 = threadIdx.x, a1 = a0 + 1, a2 = a0 + 2, a3 = a0 + 3;
        for (int it = 0; it < (1 << 22); ++it) {
#pragma unroll
            for (int j = 0; j < 32; ++j) { a0 = fmaf(a0, 1.0001f, 0.5f); a1 = fmaf(a1, 1.0001f, 0.5f); a2 = fmaf(a2, 1.0001f, 0.5f); a3 = fmaf(a3, 1.0001f, 0.5f); }
            if ((it & 7) == 0 && *reinterpret_cast<volatile uint32_t*>(&sm.stop)) break;
        }
        if (a0 + a1 + a2 + a3 == 12345.0f) cycles[201] = 1;
    } else if (warp >= 4 && (BG & 7) != 0) {
        // background traffic of the kind the attention kernels have beside their products
        const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
        const uint32_t mine = smem_u32(sm.scratch) + (threadIdx.x & 127) * 4u;
        uint32_t acc = 0;
        for (int it = 0; it < (1 << 22); ++it) {
            if (BG & 1) {       // tensor-memory loads of 32 columns (columns 384..511, nobody writes them)
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem + lane_base + 384u + 32u * uint32_t(it & 3), v);
                tmem_ld_wait();
                acc ^= v[it & 31];
            }
            if (BG & 2) {       // shared-memory stores, 128 bytes per warp instruction
#pragma unroll
                for (int j = 0; j < 16; ++j) asm volatile("st.shared.b32 [%0], %1;" :: "r"(mine + uint32_t(j) * 512u), "r"(acc + j) : "memory");
            }
            if (BG & 4) {       // tensor-memory stores of 16 columns
                uint32_t w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) w[j] = acc + j;
                tmem_st_32x32b_x16(tmem + lane_base + 448u + 16u * uint32_t(it & 3), w);
                tmem_st_wait();
            }
            if ((it & 15) == 0 && *reinterpret_cast<volatile uint32_t*>(&sm.stop)) break;
        }
        if (acc == 0x12345678u) cycles[200] = acc;
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
template <int N, int V, int BG = 0>
void run(const char* name, unsigned long long* d_cycles, int sms) {
    static uint8_t* src = nullptr;
    if (!src) { cudaMalloc(&src, 2 << 20); cudaMemset(src, 0, 2 << 20); }
    const int rounds = 2048;
    cudaFuncSetAttribute(mma_kernel<N, V, BG>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(Smem) + 1024));
    mma_kernel<N, V, BG><<<sms, 256, sizeof(Smem) + 1024>>>(d_cycles, 64, src);
    mma_kernel<N, V, BG><<<sms, 256, sizeof(Smem) + 1024>>>(d_cycles, rounds, src);
    cudaError_t e = cudaDeviceSynchronize();
    unsigned long long h[256];
    cudaMemcpy(h, d_cycles, sizeof(unsigned long long) * sms, cudaMemcpyDeviceToHost);
    double s = 0; for (int i = 0; i < sms; ++i) s += double(h[i]);
    if (V >= 9) printf("%-40s bg=%d  %8.1f cycles per half step  %s\n", name, BG, s / sms / rounds, cudaGetErrorString(e));
    else printf("%-40s bg=%d N=%3d  %7.1f cycles per MMA (ideal %d)  %s\n", name, BG, N, s / sms / (rounds * 8.0), N / 2, cudaGetErrorString(e));
}
int main() {
    int sms = 0; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    unsigned long long* d; cudaMalloc(&d, 256 * sizeof(unsigned long long));
    run<128, 0>("SS, both K-major", d, sms);  run<64, 0>("SS, both K-major", d, sms);
    run<128, 1>("SS, both MN-major", d, sms); run<64, 1>("SS, both MN-major", d, sms);
    run<128, 2>("TS, B MN-major", d, sms);    run<64, 2>("TS, B MN-major", d, sms);
    run<128, 3>("TS, B K-major", d, sms);     run<64, 3>("TS, B K-major", d, sms);
    run<64, 9, 0>("half-step sequence (32 products)", d, sms); run<64, 9, 7>("half-step sequence + background", d, sms);
    run<128, 10, 0>("same work as N=128 products (20)", d, sms);
    run<128, 0, 192>("SS K-major + FMA warps, converged issuer", d, sms); run<64, 0, 192>("SS K-major + FMA warps, converged issuer", d, sms);
    run<128, 0, 128>("SS K-major, converged issuer", d, sms);
    run<64, 9, 64>("half-step sequence + FMA warps", d, sms); run<128, 0, 64>("SS K-major + FMA warps", d, sms); run<64, 0, 64>("SS K-major + FMA warps", d, sms);
    run<128, 0, 32>("SS K-major + bulk loads", d, sms); run<64, 0, 32>("SS K-major + bulk loads", d, sms);
    run<128, 2, 32>("TS MN + bulk loads", d, sms); run<64, 1, 39>("SS MN/MN + bulk loads + all", d, sms);
    run<128, 0, 8>("SS K-major + commit per 8", d, sms); run<64, 0, 8>("SS K-major + commit per 8", d, sms);
    run<128, 0, 24>("SS K-major + commit + overwrite", d, sms); run<64, 0, 24>("SS K-major + commit + overwrite", d, sms);
    run<128, 0, 1>("SS K-major + tmem loads", d, sms); run<64, 0, 1>("SS K-major + tmem loads", d, sms);
    run<128, 0, 2>("SS K-major + st.shared", d, sms);  run<64, 0, 2>("SS K-major + st.shared", d, sms);
    run<128, 0, 4>("SS K-major + tmem stores", d, sms); run<64, 0, 4>("SS K-major + tmem stores", d, sms);
    run<128, 2, 1>("TS MN + tmem loads", d, sms);      run<128, 2, 4>("TS MN + tmem stores", d, sms);
    run<128, 2, 7>("TS MN + all three", d, sms);       run<64, 1, 7>("SS MN/MN + all three", d, sms);
    return 0;
}
