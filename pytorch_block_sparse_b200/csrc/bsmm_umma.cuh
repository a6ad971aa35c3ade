// Launchers of the tcgen05 / TMA kernels and of the plan builder they consume.
#pragma once
#include "bsmm_common.cuh"

namespace bsmm {

// One plan entry per non-zero block, grouped by BSMM_PLAN_GROUP consecutive output block-rows and
// ordered inside a group by (inner block index, row-in-group).
struct __align__(16) PlanEntry {
    int32_t inner;    // block index along the contraction axis (selects the activation slab)
    int32_t slot;     // position of the block in `data` / the packed images
    int32_t row;      // output block-row inside the group, 0..BSMM_PLAN_GROUP-1
    int32_t flags;    // bit 0: first entry of its slab, bit 1: last entry of its slab
};
constexpr int32_t kPlanFirst = 1, kPlanLast = 2;

// Plan buffer: [group offsets: n_groups + 1 int32, padded to 16 B][entries: nnz PlanEntry]
__host__ __device__ constexpr int64_t plan_groups(int64_t n_out_blocks) {
    return (n_out_blocks + BSMM_PLAN_GROUP - 1) / BSMM_PLAN_GROUP;
}
__host__ __device__ constexpr int64_t plan_entries_offset(int64_t n_out_blocks) {
    return ((plan_groups(n_out_blocks) + 1) * 4 + 15) / 16 * 16;
}
__host__ __device__ constexpr int64_t plan_bytes(int64_t n_out_blocks, int64_t nnz) {
    return plan_entries_offset(n_out_blocks) + (nnz > 0 ? nnz : 1) * (int64_t)sizeof(PlanEntry);
}

cudaError_t launch_build_plan(const int32_t* ptr, const int32_t* idx, int64_t n_out_blocks, int64_t nnz, void* plan,
                              cudaStream_t stream);

cudaError_t launch_dsd_umma(const void* a, int64_t m, int64_t k, int64_t nnz, const void* packed, const void* plan,
                            int64_t n, void* out, const float* bias, uint32_t precision, bool dgrad,
                            bool out_colmajor, cudaStream_t stream);

int64_t sddmm_umma_workspace_bytes(int64_t rows, int64_t cols, int64_t tokens, int64_t nnz, uint32_t precision);
cudaError_t launch_sddmm_umma(const void* a, const void* b, int64_t rows, int64_t cols, int64_t tokens,
                              float* sparse_c, const int32_t* blocks, int64_t nnz, float* block_sumsq,
                              void* workspace, uint32_t precision, cudaStream_t stream);

// Reads (and optionally clears) the sticky device status word: non-zero once a kernel gave up on
// a bounded wait.  Synchronizes the device.
cudaError_t read_device_status(unsigned int* status, bool clear);

}  // namespace bsmm
