// extern "C" entry points of libbsmm_b200.so: argument validation and kernel selection.
#include "bsmm_common.cuh"
#include "bsmm_umma.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_status(cudaError_t err) {
    if (err == cudaSuccess) return BSMM_OK;
    g_last_cuda_error = static_cast<int>(err);
    return BSMM_ERR_CUDA;
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// The launchers report cudaGetLastError() after their launches.  A non-sticky error left behind by an
// earlier runtime call of the host program (its own probing of pointers, for instance) would be blamed on
// them, so every entry point that launches starts from a clean error state.
void forget_earlier_errors() { (void)cudaGetLastError(); }

}  // namespace

extern "C" {

int bsmm_abi_version(void) { return BSMM_ABI_VERSION; }

const char* bsmm_status_string(int status) {
    switch (status) {
        case BSMM_OK: return "ok";
        case BSMM_ERR_INVALID_ARGUMENT: return "invalid argument (null/misaligned pointer, negative size, or size not a multiple of 32)";
        case BSMM_ERR_UNSUPPORTED: return "unsupported flag combination";
        case BSMM_ERR_CUDA: return "CUDA error (see bsmm_last_cuda_error)";
        case BSMM_ERR_TOO_LARGE: return "size exceeds a documented limit";
        default: return "unknown status";
    }
}

int bsmm_last_cuda_error(void) { return g_last_cuda_error; }

int bsmm_device_status(unsigned int* status, int clear) {
    if (status == nullptr) return BSMM_ERR_INVALID_ARGUMENT;
    return cuda_status(bsmm::read_device_status(status, clear != 0));
}

int bsmm_debug_trace_dsd(void* device_buffer, int block) {
    bsmm::set_dsd_trace(static_cast<long long*>(device_buffer), block);
    return BSMM_OK;
}

int64_t bsmm_packed_bytes(int64_t nnz, uint32_t precision) {
    if (nnz < 0) return -1;
    return 2 * nnz * bsmm::packed_slot_bytes(precision & BSMM_PREC_MASK);
}

int bsmm_pack_weights(const float* data, int64_t nnz, uint32_t precision, void* packed, float* block_sumsq,
                      bsmm_stream_t stream) {
    precision &= BSMM_PREC_MASK;
    if (nnz < 0 || (nnz > 0 && data == nullptr) || !aligned(data, 16)) return BSMM_ERR_INVALID_ARGUMENT;
    if (nnz > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (precision == BSMM_PREC_FP32_SIMT) {
        if (block_sumsq == nullptr) return BSMM_OK;
        return cuda_status(bsmm::launch_block_sumsq(data, nnz, block_sumsq, s));
    }
    if (!bsmm::is_umma_precision(precision)) return BSMM_ERR_UNSUPPORTED;
    if (nnz > 0 && (packed == nullptr || !aligned(packed, 256))) return BSMM_ERR_INVALID_ARGUMENT;
    return cuda_status(bsmm::launch_pack(data, nnz, precision, packed, block_sumsq, s));
}

int bsmm_plan_group(int64_t m, int64_t n_out_blocks, int64_t nnz, uint32_t precision) {
    (void)nnz;
    const bool wide_ok = !bsmm::is_split_precision(precision & BSMM_PREC_MASK);  // rows with correction terms take 64 columns
    if (m <= 0 || n_out_blocks <= 0) return wide_ok ? 8 : 6;
    // The widest tile re-uses each activation slab most; narrower tiles are only worth it when the
    // wide one would leave most of the 148 SMs without a CTA.  3xTF32 at 6 rows has room for only two
    // activation stages in tensor memory, which serialises the split warps and the MMAs: with several waves
    // of CTAs the 4-row tile (four stages) is faster at every density measured.
    const int64_t tiles = (m + 127) / 128;
    if (!wide_ok && tiles * ((n_out_blocks + 5) / 6) >= 4 * 148) return 4;
    for (int g : {8, 6}) {
        if (g == 8 && !wide_ok) continue;
        if (tiles * ((n_out_blocks + g - 1) / g) >= 148) return g;
    }
    return 4;
}

int64_t bsmm_plan_bytes(int64_t n_out_blocks, int64_t nnz, int group) {
    if (n_out_blocks < 0 || nnz < 0 || !bsmm::plan_group_valid(group)) return -1;
    return bsmm::plan_bytes(n_out_blocks, nnz, group);
}

int bsmm_build_plan(const int32_t* ptr, const int32_t* idx, int64_t n_out_blocks, int64_t nnz, int group, void* plan,
                    bsmm_stream_t stream) {
    if (n_out_blocks < 0 || nnz < 0 || ptr == nullptr || plan == nullptr || (nnz > 0 && idx == nullptr))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (!bsmm::plan_group_valid(group)) return BSMM_ERR_INVALID_ARGUMENT;
    if (!aligned(plan, 16) || !aligned(idx, 8)) return BSMM_ERR_INVALID_ARGUMENT;
    if (nnz > 0x7fffffff || n_out_blocks > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    return cuda_status(
        bsmm::launch_build_plan(ptr, idx, n_out_blocks, nnz, group, plan, static_cast<cudaStream_t>(stream)));
}

int bsmm_dsd_fused(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                   const float* data, const void* packed, const void* plan, int64_t n, void* out, const float* bias,
                   const float* residual, float* pre_activation, uint32_t flags, bsmm_stream_t stream) {
    return bsmm_dsd_multi(a, m, k, ptr, idx, nnz, data, packed, plan, n, out, 0, 0, bias, residual, pre_activation,
                          nullptr, 0, flags, stream);
}

int bsmm_allreduce_peers(float* const* bufs, int n, int rank, int64_t elems, float scale, bsmm_stream_t stream) {
    forget_earlier_errors();
    if (bufs == nullptr || n < 1 || n > 8 || rank < 0 || rank >= n || elems < 0 || (elems % 4) != 0)
        return BSMM_ERR_INVALID_ARGUMENT;
    for (int r = 0; r < n; ++r)
        if (bufs[r] == nullptr || !aligned(bufs[r], 16)) return BSMM_ERR_INVALID_ARGUMENT;
    return cuda_status(bsmm::launch_allreduce_slice(bufs, n, rank, elems, scale, static_cast<cudaStream_t>(stream)));
}

// bsmm_dsd_multi (scatter_slot < 0) and bsmm_dsd_scatter (peer_outs = the ranks' tensors of parts)
static int dsd_general(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                       const float* data, const void* packed, const void* plan, int64_t n, void* out, int64_t out_ld,
                       int64_t out_col0, const float* bias, const float* residual, float* pre_activation,
                       void* const* peer_outs, int n_peer_outs, int scatter_slot, uint32_t flags, bsmm_stream_t stream);

int bsmm_dsd_multi(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                   const float* data, const void* packed, const void* plan, int64_t n, void* out, int64_t out_ld,
                   int64_t out_col0, const float* bias, const float* residual, float* pre_activation,
                   void* const* peer_outs, int n_peer_outs, uint32_t flags, bsmm_stream_t stream) {
    return dsd_general(a, m, k, ptr, idx, nnz, data, packed, plan, n, out, out_ld, out_col0, bias, residual,
                       pre_activation, peer_outs, n_peer_outs, -1, flags, stream);
}

int bsmm_dsd_scatter(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                     const float* data, const void* packed, const void* plan, int64_t n, float* scratch,
                     void* const* parts, int n_parts, int slot, uint32_t flags, bsmm_stream_t stream) {
    if (n_parts < 1 || n_parts > 8 || slot < 0 || slot >= n_parts || parts == nullptr) return BSMM_ERR_INVALID_ARGUMENT;
    if (m <= 0 || (m % (128 * (int64_t)n_parts)) != 0 || nnz == 0 || k == 0) return BSMM_ERR_UNSUPPORTED;
    const uint32_t precision = flags & BSMM_PREC_MASK;
    if ((flags & (BSMM_DSD_OUT_COLMAJOR | BSMM_DSD_GELU | BSMM_DSD_IO_BF16)) != 0 || precision == BSMM_PREC_FP32_SIMT)
        return BSMM_ERR_UNSUPPORTED;
    return dsd_general(a, m, k, ptr, idx, nnz, data, packed, plan, n, scratch, 0, 0, nullptr, nullptr, nullptr, parts,
                       n_parts, slot, flags, stream);
}

int bsmm_sum_row_slots(const float* parts, int slots, int64_t rows, int64_t cols, float* const* outs, int n_outs,
                       int64_t out_row0, bsmm_stream_t stream) {
    forget_earlier_errors();
    if (parts == nullptr || outs == nullptr || slots < 1 || n_outs < 1 || n_outs > 8 || rows < 0 || cols < 0 ||
        (cols % 4) != 0 || out_row0 < 0 || !aligned(parts, 16))
        return BSMM_ERR_INVALID_ARGUMENT;
    for (int j = 0; j < n_outs; ++j)
        if (outs[j] == nullptr || !aligned(outs[j], 16)) return BSMM_ERR_INVALID_ARGUMENT;
    return cuda_status(bsmm::launch_sum_row_slots(parts, slots, rows, cols, outs, n_outs, out_row0,
                                                  static_cast<cudaStream_t>(stream)));
}

static int dsd_general(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
                       const float* data, const void* packed, const void* plan, int64_t n, void* out, int64_t out_ld,
                       int64_t out_col0, const float* bias, const float* residual, float* pre_activation,
                       void* const* peer_outs, int n_peer_outs, int scatter_slot, uint32_t flags, bsmm_stream_t stream) {
    forget_earlier_errors();
    const bool scatter = scatter_slot >= 0;
    if (n_peer_outs < 0 || n_peer_outs > 8 || (n_peer_outs > 0 && peer_outs == nullptr)) return BSMM_ERR_INVALID_ARGUMENT;
    if (out_ld < 0 || out_col0 < 0) return BSMM_ERR_INVALID_ARGUMENT;
    const bool placed = n_peer_outs > 0 || (out_ld != 0 && out_ld != n) || out_col0 != 0;
    const uint32_t precision = flags & BSMM_PREC_MASK;
    const bool dgrad = (flags & BSMM_DSD_DGRAD) != 0;
    const bool colmajor = (flags & BSMM_DSD_OUT_COLMAJOR) != 0;
    const bool gelu = (flags & BSMM_DSD_GELU) != 0;
    const bool io16 = (flags & BSMM_DSD_IO_BF16) != 0;
    const bool fused = gelu || residual != nullptr || pre_activation != nullptr || placed;
    if (m < 0 || n < 0 || k < 0 || nnz < 0 || (n % 32) != 0 || (k % 32) != 0) return BSMM_ERR_INVALID_ARGUMENT;
    if (m == 0 || n == 0) return BSMM_OK;
    if (ptr == nullptr || out == nullptr || (nnz > 0 && (idx == nullptr || data == nullptr || a == nullptr)))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (!aligned(a, 16) || !aligned(out, 16) || !aligned(data, 16) || !aligned(idx, 8) || !aligned(residual, 16) ||
        !aligned(pre_activation, 16) || !aligned(bias, 16) || !aligned(ptr, 4))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (dgrad && (bias != nullptr || gelu || residual != nullptr || pre_activation != nullptr)) return BSMM_ERR_UNSUPPORTED;
    if (fused && colmajor) return BSMM_ERR_UNSUPPORTED;
    if (pre_activation != nullptr && !gelu) return BSMM_ERR_UNSUPPORTED;
    if (io16 && (precision != BSMM_PREC_BF16 || colmajor || residual != nullptr || pre_activation != nullptr || nnz == 0 || k == 0))
        return BSMM_ERR_UNSUPPORTED;
    if (nnz > 0x7fffffff || n / 32 > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (precision == BSMM_PREC_FP32_SIMT) {
        if (fused) return BSMM_ERR_UNSUPPORTED;  // the epilogue fusions live in the tensor-core kernel
        if (colmajor && (m + 127) / 128 > 65535) return BSMM_ERR_TOO_LARGE;
        return cuda_status(bsmm::launch_dsd_simt(static_cast<const float*>(a), m, k, ptr, idx, data, n,
                                                 static_cast<float*>(out), bias, dgrad, colmajor, s));
    }
    if (bsmm::is_umma_precision(precision)) {
        if (k == 0 || nnz == 0) {  // nothing to contract: the CUDA-core kernel writes the zeros (+bias)
            if (fused) return BSMM_ERR_UNSUPPORTED;
            return cuda_status(bsmm::launch_dsd_simt(static_cast<const float*>(a), m, k, ptr, idx, data, n,
                                                     static_cast<float*>(out), bias, dgrad, colmajor, s));
        }
        const int group = (int)((flags >> 8) & 0xFFu);
        if (packed == nullptr || plan == nullptr || !aligned(packed, 256) || !aligned(plan, 16) ||
            !bsmm::plan_group_valid(group) || (group == 8 && bsmm::is_split_precision(precision)) ||
            (group == 5 && precision != BSMM_PREC_TF32X3))
            return BSMM_ERR_INVALID_ARGUMENT;
        bsmm::DsdEpilogue epilogue;
        epilogue.residual = residual;
        epilogue.pre_act = pre_activation;
        epilogue.activation = gelu ? 1 : 0;
        epilogue.io_bf16 = io16;
        epilogue.out_ld = out_ld;
        epilogue.out_col0 = out_col0;
        epilogue.n_peer_outs = n_peer_outs;
        epilogue.scatter_rows = scatter ? m / n_peer_outs : 0;
        epilogue.scatter_slot = scatter ? scatter_slot : 0;
        for (int i = 0; i < n_peer_outs; ++i) {
            if (!aligned(peer_outs[i], 16)) return BSMM_ERR_INVALID_ARGUMENT;
            epilogue.peer_outs[i] = peer_outs[i];
        }
        return cuda_status(bsmm::launch_dsd_umma(a, m, k, nnz, packed, plan, group, n, out, bias, precision, dgrad,
                                                 colmajor, epilogue, s));
    }
    return BSMM_ERR_UNSUPPORTED;
}

int bsmm_dsd(const void* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx, int64_t nnz,
             const float* data, const void* packed, const void* plan, int64_t n, void* out, const float* bias,
             uint32_t flags, bsmm_stream_t stream) {
    if ((flags & BSMM_DSD_GELU) != 0) return BSMM_ERR_UNSUPPORTED;  // the activation belongs to bsmm_dsd_fused
    return bsmm_dsd_fused(a, m, k, ptr, idx, nnz, data, packed, plan, n, out, bias, nullptr, nullptr, flags, stream);
}

int64_t bsmm_sddmm_plan_bytes(int64_t n_block_rows, int64_t nnz) {
    if (n_block_rows < 0 || nnz < 0) return -1;
    return bsmm::sddmm_plan_bytes(n_block_rows, nnz);
}

int bsmm_build_sddmm_plan(const int32_t* ptr, int64_t n_block_rows, int64_t nnz, void* plan, bsmm_stream_t stream) {
    if (n_block_rows < 0 || nnz < 0 || ptr == nullptr || plan == nullptr || !aligned(plan, 16))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (nnz > 0x7fffffff || n_block_rows > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    return cuda_status(bsmm::launch_build_sddmm_plan(ptr, n_block_rows, nnz, plan, static_cast<cudaStream_t>(stream)));
}

int64_t bsmm_sddmm_workspace_bytes(int64_t rows, int64_t cols, int64_t tokens, int64_t nnz, uint32_t flags) {
    if (rows < 0 || cols < 0 || tokens < 0 || nnz < 0) return -1;
    const uint32_t precision = flags & BSMM_PREC_MASK;
    if (!bsmm::is_umma_precision(precision)) return 0;
    if ((flags & (BSMM_SDDMM_A_COLMAJOR | BSMM_SDDMM_B_COLMAJOR)) != 0 && (tokens % 4) != 0) return 0;
    return bsmm::sddmm_umma_workspace_bytes(rows, cols, tokens, nnz, precision);
}

int bsmm_sddmm(const void* a, const void* b, int64_t rows, int64_t cols, int64_t tokens, float* sparse_c,
               const int32_t* blocks, int64_t nnz, const int32_t* csr_idx, const void* plan, float* block_sumsq,
               void* workspace, uint32_t flags, bsmm_stream_t stream) {
    forget_earlier_errors();
    const uint32_t precision = flags & BSMM_PREC_MASK;
    const bool a_col = (flags & BSMM_SDDMM_A_COLMAJOR) != 0;
    const bool b_col = (flags & BSMM_SDDMM_B_COLMAJOR) != 0;
    if (rows < 0 || cols < 0 || tokens < 0 || nnz < 0 || (rows % 32) != 0 || (cols % 32) != 0)
        return BSMM_ERR_INVALID_ARGUMENT;
    if (nnz == 0) return BSMM_OK;
    if (sparse_c == nullptr || blocks == nullptr || (tokens > 0 && (a == nullptr || b == nullptr)))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (!aligned(a, 16) || !aligned(b, 16) || !aligned(sparse_c, 16) || !aligned(blocks, 8) || !aligned(csr_idx, 8) ||
        !aligned(plan, 16) || !aligned(workspace, 16))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (nnz > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    if (precision != BSMM_PREC_FP32_SIMT && !bsmm::is_umma_precision(precision)) return BSMM_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool io16 = (flags & BSMM_SDDMM_IO_BF16) != 0;
    if (io16 && (precision != BSMM_PREC_BF16 || a_col || b_col)) return BSMM_ERR_UNSUPPORTED;
    if (precision != BSMM_PREC_FP32_SIMT) {
        const cudaError_t err = bsmm::launch_sddmm_umma(a, a_col, b, b_col, rows, cols, tokens, sparse_c, csr_idx, plan,
                                                        nnz, block_sumsq, workspace, precision, io16, s);
        if (err != cudaErrorNotSupported) return cuda_status(err);
        // shapes the tensor-core kernel does not take run on the CUDA-core kernel (same fp32-class result)
    }
    if (io16) return BSMM_ERR_UNSUPPORTED;  // the CUDA-core kernel reads fp32 tensors only
    return cuda_status(bsmm::launch_sddmm_simt(static_cast<const float*>(a), a_col, static_cast<const float*>(b),
                                               b_col, rows, cols, tokens, sparse_c, blocks, nnz, block_sumsq, s));
}

int bsmm_rebuild_indices(const int32_t* blocks, int64_t nnz, int64_t n_block_rows, int64_t n_block_cols,
                         int32_t* cell_slot, int32_t* row_ptr, int32_t* cols_a, int32_t* col_ptr, int32_t* rows_b,
                         int32_t* status, bsmm_stream_t stream) {
    forget_earlier_errors();
    if (nnz < 0 || n_block_rows <= 0 || n_block_cols <= 0) return BSMM_ERR_INVALID_ARGUMENT;
    if (cell_slot == nullptr || row_ptr == nullptr || col_ptr == nullptr || status == nullptr ||
        (nnz > 0 && (blocks == nullptr || cols_a == nullptr || rows_b == nullptr)))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (!aligned(blocks, 8) || !aligned(cols_a, 8) || !aligned(rows_b, 8)) return BSMM_ERR_INVALID_ARGUMENT;
    if (n_block_rows > 0x7fffffff / n_block_cols || nnz > n_block_rows * n_block_cols) return BSMM_ERR_TOO_LARGE;
    return cuda_status(bsmm::launch_rebuild_indices(blocks, nnz, n_block_rows, n_block_cols, cell_slot, row_ptr, cols_a,
                                                    col_ptr, rows_b, status, static_cast<cudaStream_t>(stream)));
}

int bsmm_select_lowest(const float* stat, int64_t n, int64_t k, int32_t* out_idx, bsmm_stream_t stream) {
    forget_earlier_errors();
    if (n < 0 || k < 0 || k > n || (k > 0 && (stat == nullptr || out_idx == nullptr))) return BSMM_ERR_INVALID_ARGUMENT;
    if (n > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    return cuda_status(bsmm::launch_select_lowest(stat, n, k, out_idx, static_cast<cudaStream_t>(stream)));
}

int bsmm_sample_free_cells(const int32_t* cell_slot, int64_t cells, int64_t n_free, int64_t k, uint64_t seed,
                           int32_t* free_cells, int32_t* out_cells, int32_t* status, bsmm_stream_t stream) {
    forget_earlier_errors();
    if (cells <= 0 || n_free < 0 || n_free > cells || k < 0 || k > n_free) return BSMM_ERR_INVALID_ARGUMENT;
    if (cell_slot == nullptr || status == nullptr || (k > 0 && (free_cells == nullptr || out_cells == nullptr)))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (cells > 0x7fffffff) return BSMM_ERR_TOO_LARGE;
    return cuda_status(bsmm::launch_sample_free_cells(cell_slot, cells, n_free, k, seed, free_cells, out_cells, status,
                                                      static_cast<cudaStream_t>(stream)));
}

int bsmm_move_blocks(int32_t* blocks, const int32_t* slots, const int32_t* cells, int64_t k, int64_t n_block_cols,
                     int64_t nnz, int32_t* status, bsmm_stream_t stream) {
    forget_earlier_errors();
    if (k < 0 || nnz < 0 || n_block_cols <= 0 || status == nullptr ||
        (k > 0 && (blocks == nullptr || slots == nullptr || cells == nullptr)))
        return BSMM_ERR_INVALID_ARGUMENT;
    if (!aligned(blocks, 8)) return BSMM_ERR_INVALID_ARGUMENT;
    return cuda_status(bsmm::launch_move_blocks(blocks, slots, cells, k, n_block_cols, nnz, status,
                                                static_cast<cudaStream_t>(stream)));
}

int bsmm_sddmm_static(const void* a, const void* b, int64_t rows, int64_t cols, int64_t tokens, float* sparse_c,
                      const int32_t* blocks, int64_t nnz, const int32_t* csr_idx, const void* plan,
                      float* block_sumsq, uint32_t flags, bsmm_stream_t stream) {
    // How much scratch would bsmm_sddmm want for this problem?  (Zero when the token axis is not split or
    // the CUDA-core kernel will run: then the static array is not touched at all.)
    const int64_t need = (csr_idx != nullptr && plan != nullptr)
                             ? bsmm_sddmm_workspace_bytes(rows, cols, tokens, nnz, flags)
                             : 0;
    if (need < 0) return BSMM_ERR_INVALID_ARGUMENT;
    if (need > (int64_t)BSMM_SDDMM_STATIC_MAX_BYTES) return BSMM_ERR_TOO_LARGE;
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // first call on this device: resolves the device address of the file-scope array
    const cudaError_t err = bsmm::sddmm_static_scratch(&scratch, &scratch_bytes);
    if (err != cudaSuccess) return cuda_status(err);
    return bsmm_sddmm(a, b, rows, cols, tokens, sparse_c, blocks, nnz, csr_idx, plan, block_sumsq,
                      need > 0 ? scratch : nullptr, flags, stream);
}

}  // extern "C"
