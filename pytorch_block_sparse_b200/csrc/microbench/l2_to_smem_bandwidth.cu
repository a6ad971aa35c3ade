// L2 -> shared memory bulk-copy bandwidth (diagnostic)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "bsmm_ptx.cuh"
using namespace bsmm::ptx;
constexpr int ST = 12; constexpr uint32_t BYTES = 16384;
__global__ void k(const uint8_t* src, size_t region, int iters, long long* out) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[ST];
    __shared__ volatile uint32_t abort_flag;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    if (threadIdx.x == 0) { for (int s = 0; s < ST; ++s) mbar_init(smem_u32(&bars[s]), 1); abort_flag = 0; fence_mbar_init(); }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    const size_t nchunks = region / BYTES;
    size_t c = ((size_t)blockIdx.x * 7919) % nchunks;
    long long t0 = clock64();
    uint32_t ph = 0; int s = 0;
    for (int i = 0; i < iters + ST; ++i) {
        const uint32_t bar = smem_u32(&bars[s]);
        if (i >= ST) { if (!mbar_wait(bar, ph, &abort_flag)) break; }
        if (i < iters && elect_one()) {
            mbar_arrive_expect_tx(bar, BYTES);
            bulk_load(base + s * BYTES, src + c * BYTES, BYTES, bar);
        }
        c += 148 * 3 + 1; if (c >= nchunks) c -= nchunks;
        if (++s == ST) { s = 0; if (i >= ST) ph ^= 1u; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = clock64() - t0;
}
int main() {
    long long* d; cudaMalloc(&d, 256 * 8);
    uint8_t* src; size_t big = (size_t)2 << 30; cudaMalloc(&src, big); cudaMemset(src, 1, big);
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, ST * BYTES + 1024);
    for (size_t region : {(size_t)32 << 20, (size_t)64 << 20, (size_t)2 << 30}) {
        const int iters = 4000;
        cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
        k<<<148, 64, ST * BYTES + 1024>>>(src, region, 200, d);
        cudaEventRecord(a);
        k<<<148, 64, ST * BYTES + 1024>>>(src, region, iters, d);
        cudaEventRecord(b);
        cudaError_t e = cudaDeviceSynchronize();
        float ms; cudaEventElapsedTime(&ms, a, b);
        printf("region %zu MiB: %.2f TB/s (%s)\n", region >> 20, 148.0 * iters * BYTES / ms / 1e9, cudaGetErrorString(e));
    }
    return 0;
}
