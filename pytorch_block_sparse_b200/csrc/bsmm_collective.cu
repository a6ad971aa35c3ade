// Kernels that finish a sum over ranks through NVLink peer mappings (symmetric memory): plain 16-byte loads and
// stores on other GPUs' buffers, no atomics, sums in rank order (every rank obtains the same bits).
//
// sum_row_slots: second half of the input gradient's all-reduce for a layer sharded by output features.  The dgrad kernel's
// epilogue has stored every rank's partial tiles into per-source slots on the rank that owns the tile's rows
// (reduce-scatter by rows, bsmm_umma.cu); this kernel adds the slots of the rows this rank owns in a fixed order
// (deterministic) and stores the sums into every rank's full gradient tensor, the other GPUs' through NVLink peer
// mappings (plain 16-byte stores).  HBM-bound: slots x rows x cols x 4 bytes read, n_outs x rows x cols x 4 written.
//
// allreduce_slice: in-place all-reduce of one buffer per rank (the nnz-block weight gradient of token data
// parallelism, a few MB): rank r adds slice r of every rank's buffer and stores the sum into slice r of every
// rank's buffer.  One small grid (no shared memory, 256 threads per CTA) that fits beside the persistent
// tensor-core kernels, so it can run on a side stream under the input-gradient product.
//
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

struct PeerBufs {
    float4* ptr[kMaxOuts];
};

__global__ void __launch_bounds__(256)
allreduce_slice_kernel(const PeerBufs bufs, int n, int64_t begin4, int64_t end4, float scale) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < end4; i += step) {
        float4 v[kMaxOuts];
#pragma unroll
        for (int r = 0; r < kMaxOuts; ++r)  // all loads in flight before the first addition
            if (r < n) v[r] = __ldcg(bufs.ptr[r] + i);
        float4 acc = v[0];
#pragma unroll
        for (int r = 1; r < kMaxOuts; ++r)
            if (r < n) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
#pragma unroll
        for (int r = 0; r < kMaxOuts; ++r)
            if (r < n) bufs.ptr[r][i] = acc;
    }
}

}  // namespace

cudaError_t launch_allreduce_slice(float* const* bufs, int n, int rank, int64_t elems, float scale, cudaStream_t stream) {
    if (n < 1 || n > kMaxOuts || rank < 0 || rank >= n || elems < 0 || (elems % 4) != 0) return cudaErrorInvalidValue;
    const int64_t total4 = elems / 4;
    const int64_t per = (total4 + n - 1) / n;
    const int64_t begin4 = per * rank < total4 ? per * rank : total4;
    const int64_t end4 = begin4 + per < total4 ? begin4 + per : total4;
    if (end4 <= begin4) return cudaSuccess;
    PeerBufs b;
    for (int r = 0; r < kMaxOuts; ++r) b.ptr[r] = r < n ? reinterpret_cast<float4*>(bufs[r]) : nullptr;
    const int64_t want = (end4 - begin4 + 255) / 256;
    const unsigned grid = (unsigned)(want < 128 ? want : 128);  // a small grid: it shares the GPU with a running product
    allreduce_slice_kernel<<<grid, 256, 0, stream>>>(b, n, begin4, end4, scale);
    return cudaGetLastError();
}

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
