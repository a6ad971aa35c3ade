// Producer/consumer hand-off through a ring of mbarriers on one SM: cycles per entry for the flavours of wait and
// arrive the kernels could use (try_wait, test_wait polling, relaxed forms, bounded mbar_wait), ring depths 1-16.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "bsmm_ptx.cuh"
using namespace bsmm::ptx;
constexpr int N = 4096;
__device__ __forceinline__ bool try_relaxed(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.relaxed.cta.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void arrive_relaxed(uint32_t bar) {
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__shared__ volatile uint32_t g_abort;
// Every flavour of wait is bounded: after kSpinLimit polls it raises g_abort and returns, and every waiter leaves
// as soon as it sees the flag (the timing of such a run is meaningless and the report says so).
constexpr int kSpinLimit = 1 << 22;
template <int MODE> __device__ __forceinline__ void waitf(uint32_t bar, uint32_t parity) {
    if (MODE == 3) { mbar_wait(bar, parity, &g_abort); return; }
    if (MODE == 4) {
        if (mbar_try_wait(bar, parity)) return;
        for (int outer = 0; outer < kSpinLimit / 64 && g_abort == 0; ++outer) {
#pragma unroll 1
            for (int i = 0; i < 64; ++i) if (mbar_try_wait(bar, parity)) return;
        }
        g_abort = 1;
        return;
    }
    for (int i = 0; i < kSpinLimit; ++i) {
        const bool done = MODE == 0 ? mbar_try_wait(bar, parity) : MODE == 1 ? mbar_test_wait(bar, parity) : try_relaxed(bar, parity);
        if (done) return;
        if ((i & 1023) == 1023 && g_abort != 0) return;
    }
    g_abort = 1;
}
template <int MODE> __device__ __forceinline__ void arrivef(uint32_t bar) {
    if (MODE == 2) arrive_relaxed(bar); else mbar_arrive(bar);
}
template <int MODE, int ST, bool ELECT>
__global__ void k(long long* out, int slot) {
    __shared__ __align__(8) uint64_t bars[64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto full = [&](int s) { return smem_u32(&bars[s]); };
    auto empty = [&](int s) { return smem_u32(&bars[32 + s]); };
    if (threadIdx.x == 0) { g_abort = 0; for (int s = 0; s < ST; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); } fence_mbar_init(); }
    __syncthreads();
    long long t0 = clock64();
    int ws = 0; uint32_t wph = 0;
    if (warp == 0) {
        for (int e = 0; e < N; ++e) {
            waitf<MODE>(empty(ws), wph ^ 1u);
            if (ELECT) { if (elect_one()) arrivef<MODE>(full(ws)); } else { if (lane == 0) arrivef<MODE>(full(ws)); }
            if (++ws == ST) { ws = 0; wph ^= 1u; }
        }
    } else if (warp == 1) {
        for (int e = 0; e < N; ++e) {
            waitf<MODE>(full(ws), wph);
            if (ELECT) { if (elect_one()) arrivef<MODE>(empty(ws)); } else { if (lane == 0) arrivef<MODE>(empty(ws)); }
            if (++ws == ST) { ws = 0; wph ^= 1u; }
        }
    }
    long long t1 = clock64();
    if (lane == 0 && warp == 0) out[slot] = g_abort != 0 ? -1 : t1 - t0;  // -1: a wait ran out
}
int main() {
    long long* d; cudaMalloc(&d, 64 * 8); cudaMemset(d, 0, 64 * 8);
    int slot = 0;
    auto report = [&](const char* name) {
        cudaError_t e = cudaDeviceSynchronize();
        long long h[64]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
        printf("%-44s %.1f clk/entry (%s)\n", name, (double)h[slot] / N, cudaGetErrorString(e)); ++slot;
    };
    k<0, 16, true><<<1, 64>>>(d, slot); report("try_wait, 16 stages, elect");
    k<3, 16, true><<<1, 64>>>(d, slot); report("mbar_wait (bounded), 16 stages, elect");
    k<4, 16, true><<<1, 64>>>(d, slot); report("try + nested loop of try, 16 stages, elect");
    k<3, 16, false><<<1, 64>>>(d, slot); report("mbar_wait (bounded), 16 stages, lane 0");
    k<0, 1, true><<<1, 64>>>(d, slot); report("try_wait, 1 stage, elect");
    k<1, 16, true><<<1, 64>>>(d, slot); report("test_wait spin, 16 stages, elect");
    k<1, 2, true><<<1, 64>>>(d, slot); report("test_wait spin, 2 stages, elect");
    k<2, 16, true><<<1, 64>>>(d, slot); report("relaxed try_wait + arrive, 16 stages, elect");
    k<2, 2, true><<<1, 64>>>(d, slot); report("relaxed try_wait + arrive, 2 stages, elect");
    k<0, 16, false><<<1, 64>>>(d, slot); report("try_wait, 16 stages, lane 0 arrives");
    k<2, 16, false><<<1, 64>>>(d, slot); report("relaxed, 16 stages, lane 0 arrives");
    cudaFuncSetAttribute(k<3, 16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 140000);
    k<3, 16, true><<<1, 64, 140000>>>(d, slot); report("mbar_wait, 16 stages, elect, 140 KB dyn smem");
    k<3, 16, true><<<1, 64, 60000>>>(d, slot); report("mbar_wait, 16 stages, elect, 60 KB dyn smem");
    k<3, 16, true><<<1, 352, 140000>>>(d, slot); report("mbar_wait, 16 st, elect, 140 KB, 352 thr");
    return 0;
}
