// Second half of the input gradient's all-reduce for a layer sharded by output features.  The dgrad kernel's
// epilogue has stored every rank's partial tiles into per-source slots on the rank that owns the tile's rows
// (reduce-scatter by rows, bsmm_umma.cu); this kernel adds the slots of the rows this rank owns in a fixed order
// (deterministic) and stores the sums into every rank's full gradient tensor, the other GPUs' through NVLink peer
// mappings (plain 16-byte stores).  HBM-bound: slots x rows x cols x 4 bytes read, n_outs x rows x cols x 4 written.
// The reference has no multi-GPU path (its only artefact is tests/test_data_parallel.py:11-17).
#include <cuda_runtime.h>

#include "bsmm_umma.cuh"

namespace bsmm {
namespace {

constexpr int kMaxOuts = 8;
struct SumOuts {
    float4* ptr[kMaxOuts];
};

__global__ void __launch_bounds__(256)
sum_row_slots_kernel(const float4* __restrict__ parts, int slots, int64_t slot_stride4, int64_t total4,
                     const SumOuts outs, int n_outs) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += step) {
        float4 acc = __ldcs(parts + i);
        for (int s = 1; s < slots; ++s) {
            const float4 v = __ldcs(parts + s * slot_stride4 + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        for (int j = 0; j < n_outs; ++j) outs.ptr[j][i] = acc;
    }
}

}  // namespace

cudaError_t launch_sum_row_slots(const float* parts, int slots, int64_t rows, int64_t cols, float* const* outs, int n_outs,
                                 int64_t out_row0, cudaStream_t stream) {
    if (slots < 1 || n_outs < 1 || n_outs > kMaxOuts || rows < 0 || cols < 0 || (cols % 4) != 0 || out_row0 < 0)
        return cudaErrorInvalidValue;
    const int64_t total4 = rows * cols / 4;
    if (total4 == 0) return cudaSuccess;
    SumOuts o;
    for (int j = 0; j < kMaxOuts; ++j)
        o.ptr[j] = j < n_outs ? reinterpret_cast<float4*>(outs[j] + out_row0 * cols) : nullptr;
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    const int64_t want = (total4 + 255) / 256;
    const int64_t cap = (int64_t)sms * 8;  // eight resident CTAs of 256 threads per SM, grid-stride beyond that
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    sum_row_slots_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(parts), slots, total4, total4, o, n_outs);
    return cudaGetLastError();
}

}  // namespace bsmm
