// Launch-plan builder for the tensor-core dsd kernel.
//
// The kernel owns a tile of 128 tokens x `group` (4, 5, 6 or 8) output block-rows and walks the
// contraction axis one 32-wide activation slab at a time, so it wants the group's blocks merged
// across its rows and ordered by slab.  The CSR/CSC arrays of the reference
// (block_sparse.py:85-153) list each row's blocks in ascending inner index; the merged position of
// an entry is therefore a sum of lower bounds over the rows of its group -- no sort needed.
#include "bsmm_umma.cuh"

namespace bsmm {
namespace {

constexpr int kMaxGroup = 8;

__global__ void __launch_bounds__(128)
build_plan_kernel(const int32_t* __restrict__ ptr, const int2* __restrict__ idx, int n_out_blocks, int G,
                  int32_t* __restrict__ group_off, int32_t* __restrict__ group_slabs,
                  PlanEntry* __restrict__ entries) {
    __shared__ int rp[kMaxGroup + 1];
    __shared__ int slabs;
    if (threadIdx.x == 0) slabs = 0;
    const int g = blockIdx.x;
    const int r0 = g * G;
    const int nrows = min(G, n_out_blocks - r0);
    if (threadIdx.x <= G) rp[threadIdx.x] = ptr[r0 + min((int)threadIdx.x, nrows)];
    __syncthreads();
    const int base = rp[0], end = rp[nrows];
    if (threadIdx.x == 0) {
        group_off[g] = base;
        if (g == gridDim.x - 1) group_off[g + 1] = end;
    }
    for (int e = base + threadIdx.x; e < end; e += blockDim.x) {
        const int2 ent = idx[e];
        int r = 0;
        while (r + 1 < nrows && rp[r + 1] <= e) ++r;
        int rank = 0;
        bool before = false, after = false, warp_after = false;
        uint32_t warps_present = 0;
        for (int q = 0; q < nrows; ++q) {
            int lo = rp[q], hi = rp[q + 1];
            const int row_end = hi;
            while (lo < hi) {  // first entry of row q whose inner index is >= ent.x
                const int mid = (lo + hi) >> 1;
                if (idx[mid].x < ent.x) lo = mid + 1; else hi = mid;
            }
            rank += lo - rp[q];
            const bool present = lo < row_end && idx[lo].x == ent.x;
            if (present && q < r) { ++rank; before = true; }
            if (present && q > r) after = true;
            if (present && q > r && (q % kDsdMmaWarps) == (r % kDsdMmaWarps)) warp_after = true;
            if (present || q == r) warps_present |= 1u << (q % kDsdMmaWarps);
        }
        PlanEntry pe;
        pe.inner = ent.x;
        pe.slot = ent.y;
        pe.row = r;
        // promote the row's partial sum after every kDrainEvery-th block of the row and after its last one
        const int ord = e - rp[r];
        const bool drain = ((ord + 1) % kDrainEvery) == 0 || e + 1 == rp[r + 1];
        const int idle = kDsdMmaWarps - __popc(warps_present);
        pe.flags = (before ? 0 : kPlanFirst) | (after ? 0 : kPlanLast | (idle << kPlanIdleShift)) |
                   (drain ? kPlanDrain : 0) | (warp_after ? 0 : kPlanWarpLast) | (e + 1 == rp[r + 1] ? kPlanRowEnd : 0);
        entries[base + rank] = pe;
        if (!before) atomicAdd(&slabs, 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) group_slabs[g] = slabs;
}

}  // namespace

cudaError_t launch_build_plan(const int32_t* ptr, const int32_t* idx, int64_t n_out_blocks, int64_t nnz, int group,
                              void* plan, cudaStream_t stream) {
    (void)nnz;
    if (!plan_group_valid(group)) return cudaErrorInvalidValue;
    const int64_t groups = plan_groups(n_out_blocks, group);
    if (groups == 0) return cudaSuccess;
    int32_t* group_off = static_cast<int32_t*>(plan);
    int32_t* group_slabs = group_off + groups + 1;
    PlanEntry* entries =
        reinterpret_cast<PlanEntry*>(static_cast<uint8_t*>(plan) + plan_entries_offset(n_out_blocks, group));
    build_plan_kernel<<<(unsigned)groups, 128, 0, stream>>>(ptr, reinterpret_cast<const int2*>(idx), (int)n_out_blocks,
                                                            group, group_off, group_slabs, entries);
    return cudaGetLastError();
}

}  // namespace bsmm
