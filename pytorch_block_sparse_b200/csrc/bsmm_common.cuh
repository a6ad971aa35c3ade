// Shared declarations of the engine's translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "bsmm_b200.h"

namespace bsmm {

constexpr int kBlock = 32;             // block edge (the reference's OPTIMIZED_BLOCK_SIZE)
constexpr int kBlockElems = 32 * 32;   // 1024 values, 4 KiB fp32 per slot

// tf32 operand image of one 32 (mn) x 32 (k) block, hi and lo parts interleaved per k-chunk:
// K-major, un-swizzled UMMA canonical layout of 8 x (16 B) core matrices,
//   k-chunk (4 values of k) stride = leading byte offset = 1024 B: [hi: 4 mn-groups][lo: 4 mn-groups],
//   mn-group (8 rows) stride = stride byte offset = 128 B.
// Read with N = 64 from the image start, the MMA sees the operand [hi rows 0..31 ; lo rows 0..31];
// read with N = 32 it sees the hi part alone.
__host__ __device__ constexpr uint32_t image32_offset(uint32_t mn, uint32_t k, uint32_t lo_part) {
    return (k >> 2) * 1024u + lo_part * 512u + (mn >> 3) * 128u + (mn & 7u) * 16u + (k & 3u) * 4u;
}
constexpr uint32_t kImage32Bytes = 8192;       // hi + lo
constexpr uint32_t kImage32Lbo = 1024;
constexpr uint32_t kImage32Sbo = 128;
constexpr uint32_t kImage32StepBytes = 2048;   // one MMA k-step = 8 values of k = two k-chunks

// bf16 operand image of one 32 x 32 block: core-matrix rows hold 8 values of k; k-chunks 512 B apart.
__host__ __device__ constexpr uint32_t image16_offset(uint32_t mn, uint32_t k) {
    return (k >> 3) * 512u + (mn >> 3) * 128u + (mn & 7u) * 16u + (k & 7u) * 2u;
}
constexpr uint32_t kImage16Bytes = 2048;
constexpr uint32_t kImage16Lbo = 512;
constexpr uint32_t kImage16Sbo = 128;
constexpr uint32_t kImage16StepBytes = 1024;   // one MMA k-step = 16 values of k = two k-chunks

// bf16 hi | lo operand image of one 32 x 32 block (the bf16 pair splitting of BSMM_PREC_BF16X3): per k-chunk of 8
// values [hi: 4 mn-groups][lo: 4 mn-groups], 1 KiB; an N = 64 instruction sees [hi rows ; lo rows], an N = 32
// instruction the hi part.
__host__ __device__ constexpr uint32_t image16x3_offset(uint32_t mn, uint32_t k, uint32_t lo_part) {
    return (k >> 3) * 1024u + lo_part * 512u + (mn >> 3) * 128u + (mn & 7u) * 16u + (k & 7u) * 2u;
}
constexpr uint32_t kImage16x3Bytes = 4096;
constexpr uint32_t kImage16x3Lbo = 1024;
constexpr uint32_t kImage16x3Sbo = 128;
constexpr uint32_t kImage16x3StepBytes = 2048;   // one MMA k-step = 16 values of k = two k-chunks

// tensor-core arithmetic that reads the tf32 images
__host__ __device__ constexpr bool is_tf32_precision(uint32_t precision) {
    return precision == BSMM_PREC_TF32X3 || precision == BSMM_PREC_TF32;
}

// any of the tensor-core precisions
__host__ __device__ constexpr bool is_umma_precision(uint32_t precision) {
    return is_tf32_precision(precision) || precision == BSMM_PREC_BF16 || precision == BSMM_PREC_BF16X3;
}
// an output row keeps main and correction terms apart: 64 tensor-memory columns instead of 32
__host__ __device__ constexpr bool is_split_precision(uint32_t precision) {
    return precision == BSMM_PREC_TF32X3 || precision == BSMM_PREC_BF16X3;
}

// Packed-weight buffer layout: [fwd images: nnz][dgrad images: nnz]
__host__ __device__ constexpr int64_t packed_slot_bytes(uint32_t precision) {
    return is_tf32_precision(precision)   ? (int64_t)kImage32Bytes
         : precision == BSMM_PREC_BF16    ? (int64_t)kImage16Bytes
         : precision == BSMM_PREC_BF16X3  ? (int64_t)kImage16x3Bytes
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

// pattern maintenance (bsmm_pattern.cu)
cudaError_t launch_rebuild_indices(const int32_t* blocks, int64_t nnz, int64_t n_rows, int64_t n_cols,
                                   int32_t* cell_slot, int32_t* row_ptr, int32_t* cols_a, int32_t* col_ptr,
                                   int32_t* rows_b, int32_t* status, cudaStream_t stream);
cudaError_t launch_select_lowest(const float* stat, int64_t n, int64_t k, int32_t* out, cudaStream_t stream);
cudaError_t launch_sample_free_cells(const int32_t* cell_slot, int64_t cells, int64_t n_free, int64_t k, uint64_t seed,
                                     int32_t* free_cells, int32_t* out_cells, int32_t* status, cudaStream_t stream);
cudaError_t launch_move_blocks(int32_t* blocks, const int32_t* slots, const int32_t* cells, int64_t k, int64_t n_cols,
                               int64_t nnz, int32_t* status, cudaStream_t stream);

}  // namespace bsmm
