// Micro-benchmark 5: the dsd kernel's exact MMA sequences on an otherwise idle SM.
#include <cstdio>
#include <cuda_runtime.h>
#include "bsmm_ptx.cuh"
using namespace bsmm::ptx;

// MODE 0: x3 SS (A sw128 smem): per block 4 x (N=64 + N=32) + commit
// MODE 1: 1-pass SS: 4 x N=32 + commit
// MODE 2: x3 with A no-swizzle smem desc
// MODE 3: x3 TS (A from tensor memory)
// MODE 4: 1-pass TS
// MODE 5: x3 TS, the four N=64 instructions first, then the four N=32 ones
// MODE 6: x3 TS with the third product in bf16 (kind::f16, K = 16): 4 x N=64 tf32 + 2 x N=32 bf16
// MODE 7: bf16 TS: 2 x N=32 (K = 16)
// MODE 8: 3xTF32 TS for a PAIR of blocks of adjacent rows: 4 x (N=128 + N=64), accumulators of 128 columns
template <int MODE>
__global__ void __launch_bounds__(128, 1) bench(int blocks, long long* out) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bars[20];
    for (int i = threadIdx.x; i < 200 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(gen)[i] = 0;
    if (threadIdx.x == 0) { for (int i = 0; i < 20; ++i) mbar_init(smem_u32(&bars[i]), 1); fence_mbar_init(); }
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    fence_proxy_async_smem();
    tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x < 32) {
        constexpr uint32_t iw = make_idesc(2u, 128u, 64u, false, false);
        constexpr uint32_t in = make_idesc(2u, 128u, 32u, false, false);
        volatile uint32_t flag = 0;
        long long t0 = clock64();
        int ws = 0, xs = 0;
        for (int g = 0; g < blocks; ++g) {
            const uint32_t w = base + 131072 + (uint32_t)ws * 8192;   // W ring: 8 stages
            const uint32_t x = base + (uint32_t)xs * 32768;           // X ring: 4 stages of slab + lo
            const uint32_t d = tmem + (uint32_t)(g & 3) * 64;
            const uint64_t bd = smem_desc_noswizzle(w, 1024, 128);
            const uint64_t ad = (MODE == 2) ? smem_desc_noswizzle(x, 2048, 128) : smem_desc_sw128(x, 16, 1024);
            const uint32_t at = tmem + 256 + (uint32_t)(g & 3) * 64;
            const uint32_t bar = smem_u32(&bars[ws]);
            if (elect_one()) {
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint64_t b = bd + (uint64_t)(s * 128);
                    const uint64_t a = ad + (uint64_t)(s * 2);
                    if (MODE == 0 || MODE == 2) { mma_ss_tf32(d, a, b, iw, 1u); mma_ss_tf32(d + 32, a + 1024, b, in, 1u); }
                    if (MODE == 1) mma_ss_tf32(d, a, b, in, 1u);
                    if (MODE == 3) { mma_ts_tf32(d, at + s * 8, b, iw, 1u); mma_ts_tf32(d + 32, at + 32 + s * 8, b, in, 1u); }
                    if (MODE == 4) mma_ts_tf32(d, at + s * 8, b, in, 1u);
                    if (MODE == 5 || MODE == 6) mma_ts_tf32(d, at + s * 8, b, iw, 1u);
                }
                if (MODE == 8) {
                    constexpr uint32_t i128 = make_idesc(2u, 128u, 128u, false, false);
                    const uint32_t dp = tmem + (uint32_t)(g & 1) * 128;
                    const uint64_t bp = smem_desc_noswizzle(base + 131072 + (uint32_t)(ws & 3) * 16384, 2048, 128);
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        mma_ts_tf32(dp, at + s * 8, bp + (uint64_t)(s * 256), i128, 1u);
                        mma_ts_tf32(dp + 64, at + 32 + s * 8, bp + (uint64_t)(s * 256), iw, 1u);
                    }
                }
                if (MODE == 5) {
#pragma unroll
                    for (int s = 0; s < 4; ++s) mma_ts_tf32(d + 32, at + 32 + s * 8, bd + (uint64_t)(s * 128), in, 1u);
                }
                if (MODE == 6 || MODE == 7) {
                    constexpr uint32_t ih = make_idesc(1u, 128u, 32u, false, false);
                    const uint64_t bh = smem_desc_noswizzle(w, 512, 128);
#pragma unroll
                    for (int s = 0; s < 2; ++s) mma_ts_f16(d + 32, at + 32 + s * 8, bh + (uint64_t)(s * 64), ih, 1u);
                }
                mma_commit(bar);
            }
            if (++ws == 8) ws = 0;
            if ((g & 1) && ++xs == 4) xs = 0;
        }
        long long t1 = clock64();
        if (elect_one()) mma_commit(smem_u32(&bars[19]));
        bool ok = mbar_wait(smem_u32(&bars[19]), 0, &flag);
        long long t2 = clock64();
        if (threadIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ok ? 1 : 0; }
    }
    tc_fence_before(); __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int MODE> void run(long long* d, const char* name) {
    const int blocks = 256;
    cudaFuncSetAttribute(bench<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
    bench<MODE><<<1, 128, 210 * 1024>>>(blocks, d);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("CUDA error %s\n", cudaGetErrorString(e)); exit(1); }
    long long h[3]; cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
    printf("%-28s issue %.1f clk/block, total %.1f clk/block, ok=%lld\n", name, (double)h[0] / blocks, (double)h[1] / blocks, h[2]);
}
int main() {
    long long* d; cudaMalloc(&d, 32);
    run<0>(d, "x3 SS, A sw128"); run<1>(d, "1-pass SS, A sw128"); run<2>(d, "x3 SS, A no swizzle");
    run<3>(d, "x3 TS"); run<4>(d, "1-pass TS");
    run<5>(d, "x3 TS, wide then narrow"); run<6>(d, "x3 TS, third product bf16"); run<7>(d, "bf16 TS");
    run<8>(d, "x3 TS, pair of blocks");
    return 0;
}
