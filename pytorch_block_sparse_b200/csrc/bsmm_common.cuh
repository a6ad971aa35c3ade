// Shared declarations of the engine's translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "bsmm_b200.h"

namespace bsmm {

constexpr int kBlock = 32;             // block edge (the reference's OPTIMIZED_BLOCK_SIZE)
constexpr int kBlockElems = 32 * 32;   // 1024 values, 4 KiB fp32 per slot

// Byte offset of element (mn, k) inside one K-major, un-swizzled UMMA operand image of
// 32 (mn) x 32 (k) 32-bit values: 8x(16 B) core matrices, the four mn-groups of one
// k-chunk contiguous (SBO = 128 B), k-chunks 512 B apart (LBO = 512 B).
__host__ __device__ constexpr uint32_t image32_offset(uint32_t mn, uint32_t k) {
    return (k >> 2) * 512u + (mn >> 3) * 128u + (mn & 7u) * 16u + (k & 3u) * 4u;
}
constexpr uint32_t kImage32Bytes = 4096;
// Same for 16-bit values: core matrix rows hold 8 k-values; k-chunks 512 B apart.
__host__ __device__ constexpr uint32_t image16_offset(uint32_t mn, uint32_t k) {
    return (k >> 3) * 512u + (mn >> 3) * 128u + (mn & 7u) * 16u + (k & 7u) * 2u;
}
constexpr uint32_t kImage16Bytes = 2048;

// Packed-weight buffer layout: [fwd images: nnz][dgrad images: nnz]; one image set per slot is
//   TF32X3: hi image then lo image (8 KiB);  BF16: one image (2 KiB).
__host__ __device__ constexpr int64_t packed_slot_bytes(uint32_t precision) {
    return precision == BSMM_PREC_TF32X3 ? 2 * (int64_t)kImage32Bytes
         : precision == BSMM_PREC_BF16   ? (int64_t)kImage16Bytes
                                         : 0;
}

// launchers (one per translation unit); all return a cudaError_t
cudaError_t launch_dsd_simt(const float* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx,
                            const float* data, int64_t n, float* out, const float* bias, bool dgrad,
                            bool out_colmajor, cudaStream_t stream);
cudaError_t launch_sddmm_simt(const float* a, bool a_colmajor, const float* b, bool b_colmajor, int64_t rows,
                              int64_t cols, int64_t tokens, float* sparse_c, const int32_t* blocks, int64_t nnz,
                              float* block_sumsq, cudaStream_t stream);
cudaError_t launch_pack(const float* data, int64_t nnz, uint32_t precision, void* packed, float* block_sumsq,
                        cudaStream_t stream);
cudaError_t launch_block_sumsq(const float* data, int64_t nnz, float* block_sumsq, cudaStream_t stream);

}  // namespace bsmm
