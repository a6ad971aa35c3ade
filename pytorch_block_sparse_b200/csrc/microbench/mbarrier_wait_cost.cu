// microbenchmark of mbarrier handshakes on one SM (diagnostic, not part of the product)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "bsmm_ptx.cuh"
using namespace bsmm::ptx;
constexpr int N = 2000;
__global__ void k(long long* out, int mode, int spinners) {
    __shared__ __align__(8) uint64_t bars[8];
    __shared__ volatile uint32_t abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b0 = smem_u32(&bars[0]), b1 = smem_u32(&bars[1]), bdead = smem_u32(&bars[2]), bdone = smem_u32(&bars[3]);
    if (threadIdx.x == 0) {
        mbar_init(b0, 1); mbar_init(b1, 1); mbar_init(bdead, 1); mbar_init(bdone, 1); abort_flag = 0; fence_mbar_init();
    }
    __syncthreads();
    long long t0 = clock64();
    if (mode == 0 && warp == 0) {  // try_wait on a completed phase
        for (int i = 0; i < N; ++i) mbar_wait(b0, 1u, &abort_flag);
    } else if (mode == 1 && warp == 0) {  // elect + arrive + wait (self)
        uint32_t ph = 0;
        for (int i = 0; i < N; ++i) { if (elect_one()) mbar_arrive(b0); mbar_wait(b0, ph, &abort_flag); ph ^= 1; }
    } else if (mode == 2 || mode == 3) {  // ping-pong warp 0 <-> warp 1 (mode 3: warp 0 <-> warp 4, same SMSP)
        const int other = mode == 2 ? 1 : 4;
        uint32_t ph = 0;
        if (warp == 0) {
            for (int i = 0; i < N; ++i) { if (elect_one()) mbar_arrive(b0); mbar_wait(b1, ph, &abort_flag); ph ^= 1; }
            if (elect_one()) mbar_arrive(bdone);
        } else if (warp == other) {
            for (int i = 0; i < N; ++i) { mbar_wait(b0, ph, &abort_flag); if (elect_one()) mbar_arrive(b1); ph ^= 1; }
        } else if (warp - 5 >= 0 && warp - 5 < spinners) {
            // spinners poll a barrier that completes only when the ping-pong is over
            mbar_wait(bdone, 0, &abort_flag);
        }
    } else if (mode == 4 && warp == 0) {  // 4 shuffles + a little integer work
        int v = lane, acc = 0;
        for (int i = 0; i < N; ++i) {
            int a = __shfl_sync(0xffffffffu, v, i & 31), b = __shfl_sync(0xffffffffu, v + 1, i & 31);
            int c = __shfl_sync(0xffffffffu, v + 2, i & 31), d = __shfl_sync(0xffffffffu, v + 3, i & 31);
            acc += a ^ b ^ c ^ d; v += acc & 1;
        }
        if (acc == 12345) out[31] = acc;
    } else if (mode == 5 && warp == 0) {  // clock64 cost
        long long s = 0;
        for (int i = 0; i < N; ++i) s += clock64();
        if (s == 1) out[31] = s;
    } else if (mode == 6 && warp == 0) {  // arrive only (count 1 -> completes every time)
        for (int i = 0; i < N; ++i) if (elect_one()) mbar_arrive(b0);
    } else if (mode == 7 && warp == 0) {  // tcgen05.commit + wait, nothing outstanding
        uint32_t ph = 0;
        for (int i = 0; i < N; ++i) { if (elect_one()) mma_commit(b0); mbar_wait(b0, ph, &abort_flag); ph ^= 1; }
    }
    long long t1 = clock64();
    if (warp == 0 && lane == 0) out[mode] = (t1 - t0);
}
int main() {
    long long* d; cudaMalloc(&d, 64 * 8); cudaMemset(d, 0, 64 * 8);
    const char* names[] = {"try_wait(done)", "elect+arrive+wait self", "pingpong w0<->w1", "pingpong w0<->w4 (same SMSP)", "4 shfl", "clock64", "elect+arrive", "commit+wait self"};
    for (int spin = 0; spin <= 6; spin += 6)
    for (int mode = 0; mode < 8; ++mode) {
        if (spin && mode != 2 && mode != 3) continue;
        k<<<1, 352>>>(d, mode, spin);
        cudaError_t e = cudaDeviceSynchronize();
        long long h[64]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
        printf("%-32s spinners=%d: %.1f clk/iter (%s)\n", names[mode], spin, (double)h[mode] / N, cudaGetErrorString(e));
    }
    return 0;
}
