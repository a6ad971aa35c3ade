// tcgen05.st throughput (diagnostic)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "bsmm_ptx.cuh"
using namespace bsmm::ptx;
constexpr int N = 2000;
__global__ void k(long long* out, int warps_per_quarter, int mode) {
    __shared__ uint32_t tm;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) { tmem_alloc(smem_u32(&tm), 512); tmem_relinquish(); }
    tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tmem = tm;
    const int quarter = warp & 3, rep = warp >> 2;
    uint32_t r[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = lane * 32 + i;
    const uint32_t addr = tmem + ((uint32_t)(quarter * 32) << 16) + rep * 64;
    __syncthreads();
    long long t0 = clock64();
    if (rep < warps_per_quarter) {
        for (int i = 0; i < N; ++i) {
            if (mode == 0) { tmem_st32(addr, r); tmem_st32(addr + 32, r); tmem_wait_st(); }
            else if (mode == 1) { tmem_st32(addr, r); tmem_wait_st(); }
            else { uint32_t q[32]; tmem_ld32(addr, q); tmem_ld32(addr + 32, r); tmem_wait_ld();
#pragma unroll
                   for (int j = 0; j < 32; ++j) r[j] += q[j]; }
        }
    }
    long long t1 = clock64();
    if (lane == 0 && warp == 0) out[0] = t1 - t0;
    if (r[3] == 0xdeadbeef) out[1] = r[5];
    tc_fence_before(); __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}
int main() {
    long long* d; cudaMalloc(&d, 64);
    const char* names[] = {"2 x st.x32 + wait", "1 x st.x32 + wait", "2 x ld.x32 + wait"};
    for (int mode = 0; mode < 3; ++mode)
    for (int wpq = 1; wpq <= 4; wpq *= 2) {
        k<<<1, 128 * 4>>>(d, wpq, mode);
        cudaError_t e = cudaDeviceSynchronize();
        long long h[2]; cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
        const double bytes = (mode == 1 ? 1 : 2) * 128.0 * 32 * 4 * wpq;
        printf("%-20s warps/quarter=%d: %.1f clk/iter, %.1f B/clk (%s)\n", names[mode], wpq, (double)h[0] / N, bytes * N / h[0], cudaGetErrorString(e));
    }
    return 0;
}
