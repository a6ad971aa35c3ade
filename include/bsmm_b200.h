/*
 * C-ABI of the B200 block-sparse matmul engine (libbsmm_b200.so).
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless stated
 * otherwise, every size is in elements, and each call only enqueues work on `stream` (a
 * cudaStream_t passed as void*; NULL = the legacy default stream).  Return value:
 * BSMM_OK or one of the BSMM_ERR_* codes; bsmm_status_string() names them.
 *
 * Memory and state.  No entry point calls cudaMalloc or cudaFree; all buffers are the caller's.
 * What the library itself holds, per process: on every GPU that runs a kernel of it, a device
 * health word (4 bytes, see bsmm_device_status) and the BSMM_SDDMM_STATIC_MAX_BYTES scratch array of
 * bsmm_sddmm_static, both part of the library image; on the host, the device addresses of those two
 * symbols cached per device after the first call that needs them (plain arrays filled without a lock:
 * two threads racing on the first call both store the same value), the resolved driver entry point
 * for tensor-map encoding, the optional trace pointer of bsmm_debug_trace_dsd, and the last CUDA
 * error per thread.  Nothing else survives a call.
 *
 * Stream capture.  The first tensor-core call on a device (bsmm_dsd, bsmm_sddmm, bsmm_sddmm_static)
 * resolves a driver entry point and a symbol address, and every tensor-core call sets a kernel
 * attribute and binds the device's primary context to the calling thread (cudaFuncSetAttribute,
 * cudaSetDevice on the current device): make the first call per device before a capture begins.
 *
 * Alignment.  Activation, output, `data`, bias and workspace pointers: 16 bytes (TMA bases and 16-byte accesses);
 * `idx` and `blocks`: 8 bytes (read as int2 pairs); `ptr`: 4 bytes.  A misaligned pointer is refused with
 * BSMM_ERR_INVALID_ARGUMENT, never dereferenced.  (Allocations of torch and cudaMalloc are 256-byte aligned;
 * views and the flat buffers nn.DataParallel replicates into are not: the Python layer copies those.)
 *
 * The weight format is the reference's (pytorch_block_sparse/block_sparse.py:10-76,
 * :125-153): `data` fp32 [nnz*32, 32], slot s holding its 32x32 block transposed
 * (data[s*32+c][r] = W[R*32+r][C*32+c]); CSR `ptr`/`idx` = row_start_ends_a/cols_a,
 * CSC = col_start_ends_b/rows_b, where idx is int32 [nnz,2] = (other-axis block
 * index, slot); `blocks` int32 [2*nnz] = (block-col, block-row) per slot.
 */
#ifndef BSMM_B200_H_
#define BSMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSMM_ABI_VERSION 2

/* status codes */
#define BSMM_OK 0
#define BSMM_ERR_INVALID_ARGUMENT 1 /* null pointer, negative size, size not a multiple of 32, misaligned pointer */
#define BSMM_ERR_UNSUPPORTED 2      /* flag combination this build has no kernel for */
#define BSMM_ERR_CUDA 3             /* a CUDA call failed; bsmm_last_cuda_error() returns the cudaError_t */
#define BSMM_ERR_TOO_LARGE 4        /* size exceeds a documented limit */

/* arithmetic of a contraction (bits 0..3 of `flags`) */
#define BSMM_PREC_FP32_SIMT 0u /* exact fp32 FMA on CUDA cores (the reference's arithmetic) */
#define BSMM_PREC_TF32X3 1u    /* tcgen05 kind::tf32, 3-pass hi/lo split, fp32-class accuracy  */
#define BSMM_PREC_BF16 2u      /* tcgen05 kind::f16: operands rounded to bf16 in the kernel, fp32 accumulate; tensors stay fp32 */
#define BSMM_PREC_TF32 3u      /* tcgen05 kind::tf32, single pass (cuBLAS allow_tf32 accuracy class) */
#define BSMM_PREC_BF16X3 4u    /* fp32-class accuracy (about 5e-6): both operands are split into bf16 hi + lo parts and three
                                  kind::f16 products are added with fp32 accumulation: half the tensor-core instructions of
                                  BSMM_PREC_TF32X3 (bsmm_sddmm with a feature-major operand computes as BSMM_PREC_TF32X3);
                                  tensors stay fp32; magnitudes above bf16's largest finite value (3.39e38) round to infinity */
#define BSMM_PREC_MASK 0xFu

/* bsmm_dsd flags */
#define BSMM_DSD_DGRAD 0x10u        /* 0: out = a * W^T (CSR given); 1: out = a * W (CSC given) */
#define BSMM_DSD_OUT_COLMAJOR 0x20u /* 0: out is [m, n] row-major; 1: out is [n, m] (the reference's buffer) */
#define BSMM_DSD_GROUP(g) (((uint32_t)(g)&0xFFu) << 8) /* group size the plan was built with (tensor-core precisions) */
#define BSMM_DSD_GELU 0x40u         /* bsmm_dsd_fused only: out = gelu(a * W^T + bias + residual), erf form */
#define BSMM_DSD_IO_BF16 0x80u      /* with BSMM_PREC_BF16: `a` and `out` are bf16 tensors (row-major); bias stays fp32 */

/* bsmm_sddmm flags */
#define BSMM_SDDMM_A_COLMAJOR 0x10u /* dY given as [rows, tokens] contiguous instead of [tokens, rows] */
#define BSMM_SDDMM_B_COLMAJOR 0x20u /* X  given as [cols, tokens] contiguous instead of [tokens, cols] */
#define BSMM_SDDMM_IO_BF16 0x40u    /* with BSMM_PREC_BF16: dY and X are bf16 tensors (token-major, at least 32 tokens); sparse_c stays fp32 */

typedef void* bsmm_stream_t;

int bsmm_abi_version(void);
const char* bsmm_status_string(int status);
/* cudaError_t of the most recent BSMM_ERR_CUDA on the calling thread (0 if none). */
int bsmm_last_cuda_error(void);
/*
 * Device-side health word of the current device: 0, or non-zero once a tensor-core kernel gave up
 * on one of its bounded waits (its output is then invalid).  Synchronizes the device; `clear`
 * resets the word.  `status` is a HOST pointer.  The reference has no counterpart: its split-K
 * semaphore spins without a limit (cutlass/gemm/k_split_control.h:147-156).
 */
int bsmm_device_status(unsigned int* status, int clear);
/*
 * Diagnostics, no counterpart in the reference.  Effective only in a library built with -DBSMM_TRACE (the
 * shipped build compiles the tracing out of the kernels' control loops; the call then only stores the
 * pointer): while `device_buffer` (32 int64 on the device) is set, every tensor-core bsmm_dsd launch records
 * for its CTA number `block` how many cycles each warp role (weight / activation producers, MMA issuers,
 * split warps, drain warps) spent in each of its waits, and each role's total.
 * NULL switches tracing off.  Process-wide, not thread-safe.
 */
int bsmm_debug_trace_dsd(void* device_buffer, int block);

/*
 * Kernel-ready weight images + the per-slot sum of squares used by block_norm
 * (reference block_sparse.py:155-157; replaces the per-call transposed weight copy at
 * block_sparse.py:538-544).  `packed` must hold bsmm_packed_bytes(nnz, precision) bytes,
 * 256-byte aligned; `block_sumsq` (fp32 [nnz], may be NULL) receives sum(data[s]^2).
 * precision FP32_SIMT needs no images: packed may be NULL and only the statistic is produced.
 */
int64_t bsmm_packed_bytes(int64_t nnz, uint32_t precision);
int bsmm_pack_weights(const float* data, int64_t nnz, uint32_t precision, void* packed, float* block_sumsq,
                      bsmm_stream_t stream);

/*
 * Per-pattern launch plan of the tensor-core dsd kernel: for every group of `group`
 * consecutive output block-rows (group = 4, 5, 6 or 8; 5 with BSMM_PREC_TF32X3 only, 8 neither with it nor with BSMM_PREC_BF16X3: the kernel's tile is 128 tokens x group*32
 * columns), the group's index entries re-ordered by (inner block index, row-in-group), with the
 * points at which the kernel promotes its tensor-memory partial sums.  `plan` must hold
 * bsmm_plan_bytes(n_out_blocks, nnz, group) bytes, 16-byte aligned.  Depends only on ptr/idx
 * (each row's entries in ascending inner index, as the reference builds them); rebuild after
 * block_replace / load_state_dict.  bsmm_plan_group suggests a group size for a problem shape and
 * precision (BSMM_PREC_TF32X3 and BSMM_PREC_BF16X3 take 4 or 6: their rows occupy 64 tensor-memory columns each).
 */
int bsmm_plan_group(int64_t m, int64_t n_out_blocks, int64_t nnz, uint32_t precision);
int64_t bsmm_plan_bytes(int64_t n_out_blocks, int64_t nnz, int group);
int bsmm_build_plan(const int32_t* ptr, const int32_t* idx, int64_t n_out_blocks, int64_t nnz, int group, void* plan,
                    bsmm_stream_t stream);

/*
 * Dense x block-sparse -> dense.  Replaces blocksparse_matmul_cutlass
 * (reference native/block_sparse_native.cpp:6-16, native/block_sparse_cutlass_kernel.cu:113-150):
 *   fwd   (flags without BSMM_DSD_DGRAD): out[m, n] = a[m, k] * W^T (+ bias[n]),  W is [n, k], ptr/idx = CSR
 *   dgrad (BSMM_DSD_DGRAD)              : out[m, n] = a[m, k] * W,               W is [k, n], ptr/idx = CSC
 * a: [m, k] row-major fp32; out: fp32 (both bf16 with BSMM_DSD_IO_BF16); m is free,
 * n and k are multiples of 32.  Every output element is written (empty block-rows give zeros),
 * so `out` needs no pre-zeroing.  `data` is always required; `packed`/`plan` (and the plan's group size
 * in the flags, BSMM_DSD_GROUP) are required by the tensor-core precisions and ignored by FP32_SIMT.
 * bias may be NULL.
 */
int bsmm_dsd(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
             const float* data, const void* packed, const void* plan, int64_t n, void* out, const float* bias,
             uint32_t flags, bsmm_stream_t stream);

/*
 * bsmm_dsd with the layer's neighbours fused into the forward epilogue (tensor-core precisions, row-major
 * output, forward only).  The reference fuses nothing: its layer adds the bias in a separate pass
 * (block_sparse_linear.py:229-233) and a transformer then runs the activation or the residual add as further
 * elementwise kernels over the same [m, n] tensor.
 *   out = act(a * W^T + bias + residual)
 * residual: fp32 [m, n] row-major or NULL.  act = GELU (erf form) with BSMM_DSD_GELU, else identity.
 * pre_activation (fp32 [m, n] row-major or NULL, only with BSMM_DSD_GELU): receives a * W^T + bias + residual,
 * what a backward pass needs for the activation's derivative.  Rows of more than 48 blocks are promoted from
 * tensor memory in several parts; the parts then gather in pre_activation (in `out` itself when it is NULL) and
 * the last part reads the total back before it applies the activation.
 */
int bsmm_dsd_fused(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                   const float* data, const void* packed, const void* plan, int64_t n, void* out, const float* bias,
                   const float* residual, float* pre_activation, uint32_t flags, bsmm_stream_t stream);

/*
 * bsmm_dsd_fused writing a column slice of a wider output and, tile by tile as rows complete, the same slice of
 * further tensors -- the other GPUs' copies of the output, reached through NVLink peer mappings (plain TMA stores
 * to a peer address).  This is the forward product of a layer sharded by output features fused
 * with its all-gather: every rank's kernel delivers its columns to every rank's full-width output while it
 * computes, and a barrier across the ranks after the kernel replaces the collective.  The reference has no
 * multi-GPU path (its only artefact is a DataParallel smoke test, tests/test_data_parallel.py:11-17).
 *   out            [m, out_ld] row-major; this call writes columns out_col0 .. out_col0 + n - 1 (multiples of 32);
 *                  out_ld = 0 means n
 *   peer_outs      HOST array of n_peer_outs (<= 8) device-visible pointers to tensors laid out like `out`
 *   bias, residual, pre_activation stay [n] / [m, n] tensors of this rank's slice
 * A tile leaves for the peers only when its row is complete (rows of more than 48 blocks gather their parts in
 * the local output first).  Tensor-core precisions, row-major output only.
 */
int bsmm_dsd_multi(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                   const float* data, const void* packed, const void* plan, int64_t n, void* out, int64_t out_ld,
                   int64_t out_col0, const float* bias, const float* residual, float* pre_activation,
                   void* const* peer_outs, int n_peer_outs, uint32_t flags, bsmm_stream_t stream);

/*
 * A product fused with a reduce-scatter over rows -- the input gradient of the same sharded layer, where every
 * rank computes a partial sum of the whole [m, n] result and rank i is to own rows i * m / n_parts ... of the sum.
 *   parts     HOST array of n_parts (<= 8) device-visible pointers, one per rank in rank order, this rank's own
 *             included: rank i's tensor of parts, fp32 [n_parts][m / n_parts][n] (slot s = what rank s computed for
 *             the rows rank i owns), the other ranks' reached through NVLink peer mappings
 *   slot      this rank's index: every completed tile is stored (plain TMA store) into slot `slot` of the parts
 *             tensor of the rank that owns the tile's rows
 *   scratch   fp32 [m, n], local: rows of more than 48 blocks gather their partial sums here before the total
 *             leaves; contents unspecified afterwards
 * After a barrier across the ranks, bsmm_sum_row_slots adds a rank's slots.  m must be a multiple of
 * 128 * n_parts; tensor-core precisions, fp32 tensors; flags as for bsmm_dsd (BSMM_DSD_DGRAD or forward, no
 * bias).  Nothing is added concurrently anywhere: the result does not depend on arrival order.
 */
int bsmm_dsd_scatter(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                     const float* data, const void* packed, const void* plan, int64_t n, float* scratch,
                     void* const* parts, int n_parts, int slot, uint32_t flags, bsmm_stream_t stream);

/*
 * outs[j][(out_row0 + r) * cols + c] = sum over s < slots (in slot order) of parts[(s * rows + r) * cols + c]
 * for every j < n_outs: the second half of the all-reduce that bsmm_dsd_scatter starts -- the slots of the rows
 * this rank owns are added and the sums stored into every rank's full tensor (outs: HOST array of <= 8
 * device-visible pointers to fp32 [*, cols] tensors, peers' through NVLink mappings).  cols a multiple of 4.
 */
int bsmm_sum_row_slots(const float* parts, int slots, int64_t rows, int64_t cols, float* const* outs, int n_outs,
                       int64_t out_row0, bsmm_stream_t stream);

/*
 * In-place all-reduce (sum, times `scale`) of one fp32 buffer of `elems` elements per rank through NVLink peer
 * mappings -- the nnz-block weight gradients of token data parallelism (config 4's scheme; the reference's
 * only multi-GPU artefact is tests/test_data_parallel.py:11-17).
 *   bufs   HOST array of n (<= 8) device-visible pointers, the ranks' buffers in rank order, own included
 * This rank adds slice `rank` of every buffer in rank order and stores the result into slice `rank` of every
 * buffer (elems is cut into n slices of 16-byte granularity).  The caller synchronises the ranks before the call
 * (every buffer complete) and after it (every slice stored).  Every rank ends with the same bits.  The grid is
 * small on purpose: the kernel is meant to run on a side stream beside bsmm_dsd.  elems a multiple of 4.
 */
int bsmm_allreduce_peers(float* const* bufs, int n, int rank, int64_t elems, float scale, bsmm_stream_t stream);

/*
 * Dense^T x dense -> block-sparse (SDDMM).  Replaces blocksparse_matmul_back_cutlass
 * (reference native/block_sparse_native.cpp:18-29, native/block_sparse_cutlass_kernel_back.cu:118-160):
 *   sparse_c[s*32 + c][r] = sum_t a[t, R*32+r] * b[t, C*32+c],  (C, R) = blocks[2s], blocks[2s+1]
 * a = dY [tokens, rows], b = X [tokens, cols] (row-major unless the *_COLMAJOR flag is set),
 * rows/cols multiples of 32, tokens free.  sparse_c fp32 [nnz*32, 32] is overwritten (beta = 0).
 * `block_sumsq` (fp32 [nnz], may be NULL) receives sum(sparse_c[s]^2).
 *
 * The tensor-core kernel (BSMM_PREC_TF32X3, BSMM_PREC_TF32 or BSMM_PREC_BF16; fp32 operands in any of the four
 * contiguity combinations, at least 32 tokens, and a multiple of 4 tokens when an operand is feature-major) walks the matrix by block-rows and therefore also wants the CSR index array `csr_idx`
 * (cols_a) and the item table bsmm_build_sddmm_plan makes from the CSR offsets (row_start_ends_a); `plan`
 * must hold bsmm_sddmm_plan_bytes(n_block_rows, nnz) bytes, 16-byte aligned, and depends only on the pattern.
 * When the token axis is split over several CTAs the partial results go through `workspace`
 * (bsmm_sddmm_workspace_bytes(...) bytes, 16-byte aligned) and are summed in a fixed order.
 * With csr_idx or plan NULL, or for shapes that kernel does not take, the exact-fp32 CUDA-core kernel runs
 * instead, whatever tensor-core precision was asked for (its result is at least as accurate).
 */
int64_t bsmm_sddmm_plan_bytes(int64_t n_block_rows, int64_t nnz);
int bsmm_build_sddmm_plan(const int32_t* ptr, int64_t n_block_rows, int64_t nnz, void* plan, bsmm_stream_t stream);
int64_t bsmm_sddmm_workspace_bytes(int64_t rows, int64_t cols, int64_t tokens, int64_t nnz, uint32_t flags);
int bsmm_sddmm(const void* a, const void* b, int64_t rows, int64_t cols, int64_t tokens, float* sparse_c,
               const int32_t* blocks, int64_t nnz, const int32_t* csr_idx, const void* plan, float* block_sumsq,
               void* workspace, uint32_t flags, bsmm_stream_t stream);

/*
 * Pattern maintenance on the device (no host round trip, nothing allocated).  Together these replace the
 * tensor-op sequences of BlockSparseMatrixBase.build_indices / block_replace (reference
 * block_sparse.py:85-153, :167-219) and of MagnitudeSparseOptimizerStrategy.run (reference
 * sparse_optimizer.py:38-87).  A block position ("cell") is block-row * n_block_cols + block-col.
 * `status` is a DEVICE int32 the kernels OR flags into (the caller zeroes it and reads it when it wants
 * the check): 1 = two slots at one position, 2 = a position or slot out of range, 4 = the number of
 * empty cells differs from `n_free`.
 *
 * bsmm_rebuild_indices: from `blocks` (int32 [2*nnz], (block-col, block-row) per slot) the CSR arrays
 *   row_ptr int32 [n_block_rows+1], cols_a int32 [nnz,2] = (block-col, slot) sorted by (row, col), and the
 *   CSC arrays col_ptr int32 [n_block_cols+1], rows_b int32 [nnz,2] = (block-row, slot) sorted by (col, row)
 *   -- bit-identical to the reference's buffers for the same pattern.  `cell_slot` (int32
 *   [n_block_rows*n_block_cols], scratch and result) receives the slot at every position, -1 where empty.
 * bsmm_select_lowest: out_idx int32 [k] = the k indices of smallest stat[0..n) (ties in index order; first the
 *   elements strictly below the k-th smallest value in index order, then the ties).  Used on the per-slot sums
 *   of squares to choose the blocks a pruning step recycles.
 * bsmm_sample_free_cells: out_cells int32 [k] = k distinct empty positions of `cell_slot`, uniformly at random,
 *   a pure function of (pattern, seed): every rank of a data-parallel job that passes the same seed draws
 *   the same positions.  n_free must equal the number of empty cells (cells - nnz); free_cells int32 [n_free]
 *   is scratch.
 * bsmm_move_blocks: blocks[slots[j]] = position cells[j] for j < k (then call bsmm_rebuild_indices).
 */
int bsmm_rebuild_indices(const int32_t* blocks, int64_t nnz, int64_t n_block_rows, int64_t n_block_cols,
                         int32_t* cell_slot, int32_t* row_ptr, int32_t* cols_a, int32_t* col_ptr, int32_t* rows_b,
                         int32_t* status, bsmm_stream_t stream);
int bsmm_select_lowest(const float* stat, int64_t n, int64_t k, int32_t* out_idx, bsmm_stream_t stream);
int bsmm_sample_free_cells(const int32_t* cell_slot, int64_t cells, int64_t n_free, int64_t k, uint64_t seed,
                           int32_t* free_cells, int32_t* out_cells, int32_t* status, bsmm_stream_t stream);
int bsmm_move_blocks(int32_t* blocks, const int32_t* slots, const int32_t* cells, int64_t k, int64_t n_block_cols,
                     int64_t nnz, int32_t* status, bsmm_stream_t stream);

/*
 * bsmm_sddmm for callers that cannot allocate device memory.  No counterpart in the reference.
 *
 * Some hosts of this library may not call cudaMalloc at the point where the weight gradient is
 * needed: code running while a CUDA graph is being captured, or inside a memory pool / allocator
 * callback, an inference or training runtime that hands out all device memory up front and forbids
 * later allocation, a real-time loop that must not take the allocator's locks.  bsmm_sddmm asks such
 * a caller for a `workspace`; this variant takes none.  The partial results of the token ranges go to
 * a scratch array that is part of the library image (file scope, BSMM_SDDMM_STATIC_MAX_BYTES, held by
 * every GPU that loads the library until the process exits).
 *
 * Same arguments and result as bsmm_sddmm without `workspace`; the caller still owns every input and
 * the output.  Returns BSMM_ERR_TOO_LARGE when bsmm_sddmm_workspace_bytes(...) for the problem exceeds
 * BSMM_SDDMM_STATIC_MAX_BYTES.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current) and keeps it; make that first call before any stream capture begins.
 * All calls on one device share the one array and nothing is cleared between calls (every byte a call
 * reads it has written itself first): two calls whose kernels overlap on the GPU -- different streams,
 * or different host threads -- race on it and corrupt each other's result.  Serialise them.
 */
#define BSMM_SDDMM_STATIC_MAX_BYTES (64u << 20)
int bsmm_sddmm_static(const void* a, const void* b, int64_t rows, int64_t cols, int64_t tokens, float* sparse_c,
                      const int32_t* blocks, int64_t nnz, const int32_t* csr_idx, const void* plan,
                      float* block_sumsq, uint32_t flags, bsmm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BSMM_B200_H_ */
