// Sparsity-pattern maintenance on the device: the index work behind BlockSparseMatrix.block_replace /
// rebuild (reference block_sparse.py:85-153, :167-219) and behind one step of the magnitude pruning +
// random regrowth strategy (reference sparse_optimizer.py:38-87), without host round trips.
//
// The reference derives its five index buffers with nonzero / index_add_ / cumsum / sort on a
// [block-rows x block-cols] mask and draws the regrowth positions with a host randperm.  Here the
// matrix of block positions ("cells", X * Y of them, at most a few hundred thousand) is small enough
// that every step is one pass of a single CTA over the cells:
//
//   scatter      cell_slot[row * Y + col] = slot for every stored block (duplicate positions raise a flag)
//   compaction   CSR  = the occupied cells in row-major order    -> (block-col, slot) pairs + row offsets
//                CSC  = the occupied cells in column-major order -> (block-row, slot) pairs + column offsets
//                free = the empty cells in row-major order
//   selection    the k slots of smallest block statistic: exact radix select (4 passes of 8 bits over an
//                order-preserving integer image of the floats), ties taken in slot order
//   sampling     k distinct empty cells, uniformly: a keyed permutation of [0, free) (Feistel network with
//                cycle walking) evaluated at 0..k-1 indexes the list of empty cells.  Same seed, same state
//                -> same cells on every rank of a data-parallel job.
//
// All results are bit-identical to the reference's for the same pattern: CSR entries sorted by
// (row, col), CSC entries by (col, row), `blocks` in slot order.
#include "bsmm_common.cuh"

namespace bsmm {
namespace {

constexpr int kThreads = 1024;

// exclusive prefix of `flag` over the CTA's threads (in thread order) and the CTA's total
__device__ __forceinline__ int block_scan(int flag, int* total) {
    __shared__ int warp_sums[kThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned ballot = __ballot_sync(0xffffffffu, flag != 0);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    __syncthreads();  // warp_sums of the previous call have been read
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
        const int v = warp_sums[w];
        before += w < warp ? v : 0;
        all += v;
    }
    *total = all;
    return before + in_warp;
}

__global__ void __launch_bounds__(256)
fill_kernel(int32_t* __restrict__ p, int64_t n, int32_t value) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        p[i] = value;
}

__global__ void __launch_bounds__(256)
scatter_kernel(const int2* __restrict__ blocks, int64_t nnz, int32_t n_rows, int32_t n_cols,
               int32_t* __restrict__ cell_slot, int32_t* __restrict__ status) {
    for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < nnz; s += (int64_t)gridDim.x * blockDim.x) {
        const int2 b = blocks[s];  // (block-col, block-row)
        if (b.x < 0 || b.x >= n_cols || b.y < 0 || b.y >= n_rows) {
            atomicOr(status, 2);
            continue;
        }
        const int32_t old = atomicExch(&cell_slot[(int64_t)b.y * n_cols + b.x], (int32_t)s);
        if (old != -1) atomicOr(status, 1);  // two slots at one position
    }
}

// One CTA walks the cells in row-major (kColumnMajor = false) or column-major order and writes the occupied
// ones as (other-axis index, slot) pairs, with the offsets of every line of the walk.
template <bool kColumnMajor>
__global__ void __launch_bounds__(kThreads)
compact_kernel(const int32_t* __restrict__ cell_slot, int32_t n_rows, int32_t n_cols, int2* __restrict__ entries,
               int32_t* __restrict__ offsets) {
    const int64_t cells = (int64_t)n_rows * n_cols;
    const int32_t line = kColumnMajor ? n_rows : n_cols;  // cells per line of the walk
    int running = 0;
    for (int64_t base = 0; base < cells; base += kThreads) {
        const int64_t t = base + threadIdx.x;
        int32_t slot = -1, major = 0, minor = 0;
        if (t < cells) {
            major = (int32_t)(t / line);
            minor = (int32_t)(t - (int64_t)major * line);
            const int64_t cell = kColumnMajor ? (int64_t)minor * n_cols + major : t;
            slot = cell_slot[cell];
        }
        int total;
        const int pos = running + block_scan(slot >= 0, &total);
        if (t < cells) {
            if (minor == 0) offsets[major] = pos;
            if (slot >= 0) entries[pos] = make_int2(minor, slot);
        }
        running += total;
    }
    if (threadIdx.x == 0) offsets[kColumnMajor ? n_cols : n_rows] = running;
}

__global__ void __launch_bounds__(kThreads)
free_cells_kernel(const int32_t* __restrict__ cell_slot, int64_t cells, int32_t* __restrict__ free_cells,
                  int64_t expected, int32_t* __restrict__ status) {
    int64_t running = 0;
    for (int64_t base = 0; base < cells; base += kThreads) {
        const int64_t t = base + threadIdx.x;
        const bool is_free = t < cells && cell_slot[t] < 0;
        int total;
        const int64_t pos = running + block_scan(is_free, &total);
        if (is_free && pos < expected) free_cells[pos] = (int32_t)t;
        running += total;
    }
    if (threadIdx.x == 0 && running != expected) atomicOr(status, 4);  // the pattern does not hold nnz distinct blocks
}

__device__ __forceinline__ uint32_t order_key(float v) {  // unsigned integers in the order of the floats
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// The k smallest of stat[0..n), as indices: first those strictly below the k-th smallest value, in index order,
// then as many of the elements equal to it as are needed, in index order.
__global__ void __launch_bounds__(kThreads)
select_lowest_kernel(const float* __restrict__ stat, int64_t n, int64_t k, int32_t* __restrict__ out) {
    __shared__ unsigned int hist[256];
    __shared__ uint32_t s_prefix, s_mask;
    __shared__ long long s_remaining;
    if (threadIdx.x == 0) { s_prefix = 0; s_mask = 0; s_remaining = k; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (threadIdx.x < 256) hist[threadIdx.x] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix, mask = s_mask;
        for (int64_t i = threadIdx.x; i < n; i += kThreads) {
            const uint32_t u = order_key(stat[i]);
            if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            long long remaining = s_remaining, cum = 0;
            int bin = 0;
            for (; bin < 255; ++bin) {
                if (cum + hist[bin] >= remaining) break;
                cum += hist[bin];
            }
            s_remaining = remaining - cum;
            s_prefix = prefix | ((uint32_t)bin << shift);
            s_mask = mask | (255u << shift);
        }
        __syncthreads();
    }
    const uint32_t threshold = s_prefix;        // image of the k-th smallest value
    const long long ties = s_remaining;         // elements equal to it that belong to the result
    const long long below = k - ties;
    long long run_lt = 0, run_eq = 0;
    for (int64_t base = 0; base < n; base += kThreads) {
        const int64_t i = base + threadIdx.x;
        const uint32_t u = i < n ? order_key(stat[i]) : 0xffffffffu;
        const bool lt = i < n && u < threshold, eq = i < n && u == threshold;
        int total_lt, total_eq;
        const long long p_lt = run_lt + block_scan(lt, &total_lt);
        const long long p_eq = run_eq + block_scan(eq, &total_eq);
        if (lt) out[p_lt] = (int32_t)i;
        if (eq && p_eq < ties) out[below + p_eq] = (int32_t)i;
        run_lt += total_lt;
        run_eq += total_eq;
    }
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {  // integer finaliser (murmur3)
    x ^= x >> 16; x *= 0x85ebca6bu; x ^= x >> 13; x *= 0xc2b2ae35u; x ^= x >> 16;
    return x;
}

// A permutation of [0, n): balanced Feistel network over 2 * half_bits bits, cycle-walked into [0, n).
__device__ __forceinline__ uint64_t keyed_permutation(uint64_t j, uint64_t n, int half_bits, uint64_t seed) {
    const uint32_t half_mask = (1u << half_bits) - 1u;
    uint64_t v = j;
    do {
        uint32_t l = (uint32_t)(v >> half_bits) & half_mask, r = (uint32_t)v & half_mask;
#pragma unroll
        for (int round = 0; round < 6; ++round) {
            const uint32_t f = mix32(r ^ mix32((uint32_t)seed + 0x9e3779b9u * (uint32_t)(round + 1)) ^ (uint32_t)(seed >> 32)) & half_mask;
            const uint32_t nl = r;
            r = l ^ f;
            l = nl;
        }
        v = ((uint64_t)l << half_bits) | r;
    } while (v >= n);
    return v;
}

__global__ void __launch_bounds__(256)
pick_cells_kernel(const int32_t* __restrict__ free_cells, int64_t n_free, int64_t k, uint64_t seed, int half_bits,
                  int32_t* __restrict__ out_cells) {
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < k; j += (int64_t)gridDim.x * blockDim.x)
        out_cells[j] = free_cells[keyed_permutation((uint64_t)j, (uint64_t)n_free, half_bits, seed)];
}

__global__ void __launch_bounds__(256)
move_blocks_kernel(int2* __restrict__ blocks, const int32_t* __restrict__ slots, const int32_t* __restrict__ cells,
                   int64_t k, int32_t n_cols, int64_t nnz, int32_t* __restrict__ status) {
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < k; j += (int64_t)gridDim.x * blockDim.x) {
        const int32_t slot = slots[j], cell = cells[j];
        if (slot < 0 || slot >= nnz || cell < 0) {
            atomicOr(status, 2);
            continue;
        }
        blocks[slot] = make_int2(cell % n_cols, cell / n_cols);  // (block-col, block-row)
    }
}

unsigned grid_for(int64_t n) {
    const int64_t g = (n + 255) / 256;
    return (unsigned)(g < 1 ? 1 : g > 1184 ? 1184 : g);
}

}  // namespace

cudaError_t launch_rebuild_indices(const int32_t* blocks, int64_t nnz, int64_t n_rows, int64_t n_cols,
                                   int32_t* cell_slot, int32_t* row_ptr, int32_t* cols_a, int32_t* col_ptr,
                                   int32_t* rows_b, int32_t* status, cudaStream_t stream) {
    const int64_t cells = n_rows * n_cols;
    fill_kernel<<<grid_for(cells), 256, 0, stream>>>(cell_slot, cells, -1);
    if (nnz > 0)
        scatter_kernel<<<grid_for(nnz), 256, 0, stream>>>(reinterpret_cast<const int2*>(blocks), nnz, (int32_t)n_rows,
                                                         (int32_t)n_cols, cell_slot, status);
    compact_kernel<false><<<1, kThreads, 0, stream>>>(cell_slot, (int32_t)n_rows, (int32_t)n_cols,
                                                      reinterpret_cast<int2*>(cols_a), row_ptr);
    compact_kernel<true><<<1, kThreads, 0, stream>>>(cell_slot, (int32_t)n_rows, (int32_t)n_cols,
                                                     reinterpret_cast<int2*>(rows_b), col_ptr);
    return cudaGetLastError();
}

cudaError_t launch_select_lowest(const float* stat, int64_t n, int64_t k, int32_t* out, cudaStream_t stream) {
    if (k == 0) return cudaSuccess;
    select_lowest_kernel<<<1, kThreads, 0, stream>>>(stat, n, k, out);
    return cudaGetLastError();
}

cudaError_t launch_sample_free_cells(const int32_t* cell_slot, int64_t cells, int64_t n_free, int64_t k, uint64_t seed,
                                     int32_t* free_cells, int32_t* out_cells, int32_t* status, cudaStream_t stream) {
    if (k == 0) return cudaSuccess;
    free_cells_kernel<<<1, kThreads, 0, stream>>>(cell_slot, cells, free_cells, n_free, status);
    int half_bits = 1;
    while (((uint64_t)1 << (2 * half_bits)) < (uint64_t)n_free) ++half_bits;
    pick_cells_kernel<<<grid_for(k), 256, 0, stream>>>(free_cells, n_free, k, seed, half_bits, out_cells);
    return cudaGetLastError();
}

cudaError_t launch_move_blocks(int32_t* blocks, const int32_t* slots, const int32_t* cells, int64_t k, int64_t n_cols,
                               int64_t nnz, int32_t* status, cudaStream_t stream) {
    if (k == 0) return cudaSuccess;
    move_blocks_kernel<<<grid_for(k), 256, 0, stream>>>(reinterpret_cast<int2*>(blocks), slots, cells, k, (int32_t)n_cols,
                                                        nnz, status);
    return cudaGetLastError();
}

}  // namespace bsmm
