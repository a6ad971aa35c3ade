// Launchers of the tcgen05 / TMA kernels and of the plan builders they consume.
#pragma once
#include <cuda.h>

#include "bsmm_common.cuh"

namespace bsmm {

// One plan entry per non-zero block, grouped by `group` consecutive output block-rows and ordered
// inside a group by (inner block index, row-in-group).
struct __align__(16) PlanEntry {
    int32_t inner;    // block index along the contraction axis (selects the activation slab)
    int32_t slot;     // position of the block in `data` / the packed images
    int32_t row;      // output block-row inside the group, 0..group-1
    int32_t flags;    // kPlanFirst | kPlanLast | kPlanDrain | kPlanWarpLast | idle warps << kPlanIdleShift
};
// The dsd kernel issues its MMAs from kDsdMmaWarps warps; output row r of a group belongs to warp
// r mod kDsdMmaWarps.  A slab's tensor-memory stage is released by kDsdMmaWarps arrivals: one from every warp
// with a block in the slab (after its last one), the rest from the warp that issues the slab's last block.
constexpr int kDsdMmaWarps = 4;
constexpr int32_t kPlanFirst = 1;     // first entry of its activation slab
constexpr int32_t kPlanLast = 2;      // last entry of its activation slab
constexpr int32_t kPlanDrain = 4;     // after this entry the row's tensor-memory partial sum is promoted
constexpr int32_t kPlanWarpLast = 8;  // last entry of its slab among the rows of the same MMA warp
constexpr int kPlanIdleShift = 4;     // on the slab's last entry, 2 bits: MMA warps without a block in the slab
constexpr int32_t kPlanRowEnd = 64;   // last block of its output row: the promotion after it completes the row
// Blocks of one output row accumulated in tensor memory between two promotions.  The tensor core
// adds into its fp32 accumulator with a systematic rounding error of about 2e-8 (relative) per
// accumulation.  The kernel keeps the main term (hi*hi: 4 accumulations per block) apart from the
// small correction terms, so 48 blocks cost 192 accumulations of the main term: about 4e-6.
constexpr int kDrainEvery = 48;

inline bool plan_group_valid(int group) { return group == 4 || group == 5 || group == 6 || group == 8; }

// Plan buffer: [group offsets: n_groups + 1 int32][slabs per group: n_groups int32][pad to 16 B]
//              [entries: nnz PlanEntry]
__host__ __device__ constexpr int64_t plan_groups(int64_t n_out_blocks, int group) {
    return (n_out_blocks + group - 1) / group;
}
__host__ __device__ constexpr int64_t plan_entries_offset(int64_t n_out_blocks, int group) {
    return ((2 * plan_groups(n_out_blocks, group) + 1) * 4 + 15) / 16 * 16;
}
__host__ __device__ constexpr int64_t plan_bytes(int64_t n_out_blocks, int64_t nnz, int group) {
    return plan_entries_offset(n_out_blocks, group) + (nnz > 0 ? nnz : 1) * (int64_t)sizeof(PlanEntry);
}

cudaError_t launch_build_plan(const int32_t* ptr, const int32_t* idx, int64_t n_out_blocks, int64_t nnz, int group,
                              void* plan, cudaStream_t stream);

// Optional work fused into the epilogue of the row-major forward product: out = act(a * W^T + bias + residual).
struct DsdEpilogue {
    const float* residual = nullptr;  // [m, n] row-major, added with the bias
    float* pre_act = nullptr;         // [m, n] row-major: receives a * W^T + bias + residual when an activation is applied
    int activation = 0;               // 0 none, 1 GELU (erf form)
    bool io_bf16 = false;             // `a` and `out` are bf16 tensors (BSMM_PREC_BF16, row-major output)
    int64_t out_ld = 0;               // row pitch of `out` in elements when it is wider than n (0: n)
    int64_t out_col0 = 0;             // first column of `out` this call writes (multiple of 32)
    void* peer_outs[8] = {nullptr};   // further tensors laid out like `out` (other GPUs' copies) that receive every tile
    int n_peer_outs = 0;
    // Scatter mode (scatter_rows > 0): peer_outs[i] is rank i's [n_peer_outs * scatter_rows, out_ld] tensor of
    // parts, own rank included; rank i owns the rows [i * scatter_rows, (i + 1) * scatter_rows) of the result, and
    // a completed tile is stored into slot `scatter_slot` of its owner's tensor instead of going to every peer.
    int64_t scatter_rows = 0;
    int scatter_slot = 0;
};
// out[j][(out_row0 + r) * cols + c] = sum over s < slots of parts[(s * rows + r) * cols + c]  for every j < n_outs
// in-place sum over n ranks' buffers of `elems` floats: this rank adds slice `rank` of every buffer (rank order),
// scales it and stores it into slice `rank` of every buffer
cudaError_t launch_allreduce_slice(float* const* bufs, int n, int rank, int64_t elems, float scale, cudaStream_t stream);
cudaError_t launch_sum_row_slots(const float* parts, int slots, int64_t rows, int64_t cols, float* const* outs, int n_outs,
                                 int64_t out_row0, cudaStream_t stream);
cudaError_t launch_dsd_umma(const void* a, int64_t m, int64_t k, int64_t nnz, const void* packed, const void* plan,
                            int group, int64_t n, void* out, const float* bias, uint32_t precision, bool dgrad,
                            bool out_colmajor, const DsdEpilogue& epilogue, cudaStream_t stream);

// SDDMM: item table built from the CSR offsets (one item = up to 8 blocks of one block-row)
int64_t sddmm_plan_bytes(int64_t n_rows, int64_t nnz);
cudaError_t launch_build_sddmm_plan(const int32_t* ptr, int64_t n_rows, int64_t nnz, void* plan, cudaStream_t stream);
int64_t sddmm_umma_workspace_bytes(int64_t rows, int64_t cols, int64_t tokens, int64_t nnz, uint32_t precision);
// returns cudaErrorNotSupported for shapes it does not take (fewer than 32 tokens, missing plan, a feature-major
// operand whose token count is not a multiple of 4)
cudaError_t launch_sddmm_umma(const void* a, bool a_feature_major, const void* b, bool b_feature_major, int64_t rows,
                              int64_t cols, int64_t tokens, float* sparse_c, const int32_t* csr_idx, const void* plan,
                              int64_t nnz, float* block_sumsq, void* workspace, uint32_t precision, bool io_bf16,
                              cudaStream_t stream);

// Address and size of the library's static scratch array on the current device (first call per
// device resolves the symbol).
cudaError_t sddmm_static_scratch(void** ptr, size_t* bytes);

// Diagnostics, effective only in a library built with -DBSMM_TRACE: the following dsd launches record, for CTA
// `block`, the cycles each warp role spent in each kind of wait into `device_buffer` (32 int64, see TraceSlot
// in bsmm_umma.cu); null switches it off.
void set_dsd_trace(long long* device_buffer, int block);

// 2-D tiled tensor map over a row-major [outer, inner] array.
cudaError_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                         uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle);

// The sticky device status word of the current device: non-zero once a kernel gave up on a bounded
// wait.  Kernels receive its address as a parameter.
cudaError_t device_status_address(unsigned int** addr);
// Reads (and optionally clears) it.  Synchronizes the device.
cudaError_t read_device_status(unsigned int* status, bool clear);

}  // namespace bsmm
