// Micro-benchmark 3: cycles per tcgen05.mma, fully unrolled issue (no integer work in the loop).
#include <cstdio>
#include <cuda_runtime.h>
#include "bsmm_ptx.cuh"
using namespace bsmm::ptx;

template <int N, int NACC, int KIND, int TS>
__global__ void __launch_bounds__(128, 1) bench(int iters, long long* out) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bar;
    for (int i = threadIdx.x; i < 160 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(gen)[i] = 0;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); fence_mbar_init(); }
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    fence_proxy_async_smem();
    tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = make_idesc(KIND == 0 ? 2u : 1u, 128u, (uint32_t)N, false, false);
        constexpr uint32_t bimg = N / 8 * 128 * 2;
        long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t d = tmem + (uint32_t)((j % NACC) * N);
                const uint64_t bdesc = smem_desc_noswizzle(base + (uint32_t)(j % 8) * bimg, N / 8 * 128, 128);
                if (TS) {
                    const uint32_t a_tmem = tmem + 256 + (uint32_t)(j % 4) * 8;
                    if (KIND == 0) mma_ts_tf32(d, a_tmem, bdesc, idesc, 1u); else mma_ts_f16(d, a_tmem, bdesc, idesc, 1u);
                } else {
                    const uint64_t adesc = smem_desc_noswizzle(base + 131072 + (uint32_t)(j % 4) * 4096, 2048, 128);
                    if (KIND == 0) mma_ss_tf32(d, adesc, bdesc, idesc, 1u); else mma_ss_f16(d, adesc, bdesc, idesc, 1u);
                }
            }
        }
        long long t1 = clock64();
        mma_commit(smem_u32(&bar));
        volatile uint32_t flag = 0;
        bool ok = mbar_wait(smem_u32(&bar), 0, &flag);
        long long t2 = clock64();
        out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ok ? 1 : 0;
    }
    tc_fence_before(); __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int N, int NACC, int KIND, int TS>
void run(long long* d) {
    if (NACC * N > 256) return;
    if (8 * (N / 8 * 256) > 131072) return;
    const int iters = 32;
    cudaFuncSetAttribute(bench<N, NACC, KIND, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 176 * 1024);
    bench<N, NACC, KIND, TS><<<1, 128, 176 * 1024>>>(iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("CUDA error %s\n", cudaGetErrorString(e)); exit(1); }
    long long h[3]; cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
    const double cnt = iters * 16.0;
    printf("%s %4d %4d  %s  %10.1f  %12.1f  %lld\n", KIND ? "bf16" : "tf32", N, NACC, TS ? "tmem" : "smem", h[0] / cnt, h[1] / cnt, h[2]);
}

template <int KIND, int TS>
void sweep(long long* d) {
    run<8, 1, KIND, TS>(d); run<16, 1, KIND, TS>(d); run<16, 8, KIND, TS>(d);
    run<32, 1, KIND, TS>(d); run<32, 2, KIND, TS>(d); run<32, 8, KIND, TS>(d);
    run<64, 1, KIND, TS>(d); run<64, 4, KIND, TS>(d);
    run<128, 1, KIND, TS>(d); run<128, 2, KIND, TS>(d);
    run<256, 1, KIND, TS>(d);
}

int main() {
    long long* d; cudaMalloc(&d, 32);
    printf("kind   n  nacc  A    issue_clk/mma  total_clk/mma  ok\n");
    sweep<0, 1>(d); sweep<0, 0>(d); sweep<1, 1>(d); sweep<1, 0>(d);
    return 0;
}
