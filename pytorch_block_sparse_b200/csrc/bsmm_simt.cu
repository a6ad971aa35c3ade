// Exact-fp32 CUDA-core kernels for the three contractions of one block-sparse Linear.
//
// They compute in the reference's arithmetic (fp32 FMA, fp32 accumulate; reference
// cutlass/gemm/dp_accummulate.h:90-98) straight from the reference's `data` layout, so
// they need no packed images and no plan.  They serve BSMM_PREC_FP32_SIMT and are the
// on-device cross-check of the tensor-core kernels.  The two dsd kernels are deterministic.  The
// SDDMM kernel is deterministic only when one CTA covers a block's whole token axis (few tokens or
// many blocks); otherwise it splits the tokens over CTAs that add their partial sums with float
// atomics, so its low-order bits vary from run to run (the tensor-core SDDMM sums its partials in a
// fixed order and is reproducible).
#include "bsmm_common.cuh"

namespace bsmm {
namespace {

// ---------------------------------------------------------------------------------------------
// dense x block-sparse -> dense.  One CTA: 128 tokens x one output block-row (32 columns).
//   fwd  : out[t, R*32+n] = sum over blocks (R, C) of a[t, C*32+k] * data[slot][k][n]
//   dgrad: out[t, C*32+n] = sum over blocks (R, C) of a[t, R*32+k] * data[slot][n][k]
// grid = (n/32, ceil(m/128)); 256 threads, each a 4 (token) x 4 (column) register tile.
// ---------------------------------------------------------------------------------------------
template <bool kDgrad>
__global__ void __launch_bounds__(256)
dsd_simt_kernel(const float* __restrict__ a, int64_t m, int64_t k_in, const int32_t* __restrict__ ptr,
                const int2* __restrict__ idx, const float* __restrict__ data, int64_t n_out,
                float* __restrict__ out, const float* __restrict__ bias, int out_colmajor) {
    __shared__ float As[128][33];
    __shared__ __align__(16) float Bs[32][36];

    const int tid = threadIdx.x;
    const int tx = tid & 7;   // column group
    const int ty = tid >> 3;  // token group
    const int brow = blockIdx.x;
    const int64_t tok0 = (int64_t)blockIdx.y * 128;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int beg = ptr[brow], end = ptr[brow + 1];
    for (int e = beg; e < end; ++e) {
        const int2 ent = idx[e];  // x: inner block index, y: slot
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty + 32 * i;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tok0 + r < m)
                v = *reinterpret_cast<const float4*>(a + (tok0 + r) * k_in + (int64_t)ent.x * 32 + tx * 4);
            As[r][tx * 4 + 0] = v.x;
            As[r][tx * 4 + 1] = v.y;
            As[r][tx * 4 + 2] = v.z;
            As[r][tx * 4 + 3] = v.w;
        }
        {
            const float4 v = *reinterpret_cast<const float4*>(data + (int64_t)ent.y * kBlockElems + ty * 32 + tx * 4);
            if (!kDgrad) {
                *reinterpret_cast<float4*>(&Bs[ty][tx * 4]) = v;  // Bs[k][n] = tile[k][n]
            } else {
                Bs[tx * 4 + 0][ty] = v.x;  // Bs[k][n] = tile[n][k]
                Bs[tx * 4 + 1][ty] = v.y;
                Bs[tx * 4 + 2][ty] = v.z;
                Bs[tx * 4 + 3][ty] = v.w;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            float av[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[ty * 4 + i][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[i][0] = fmaf(av[i], b4.x, acc[i][0]);
                acc[i][1] = fmaf(av[i], b4.y, acc[i][1]);
                acc[i][2] = fmaf(av[i], b4.z, acc[i][2]);
                acc[i][3] = fmaf(av[i], b4.w, acc[i][3]);
            }
        }
        __syncthreads();
    }

    const int64_t col0 = (int64_t)brow * 32 + tx * 4;
    float bv[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = bias[col0 + j];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t t = tok0 + ty * 4 + i;
        if (t >= m) continue;
        if (!out_colmajor) {
            float4 v = make_float4(acc[i][0] + bv[0], acc[i][1] + bv[1], acc[i][2] + bv[2], acc[i][3] + bv[3]);
            *reinterpret_cast<float4*>(out + t * n_out + col0) = v;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) out[(col0 + j) * m + t] = acc[i][j] + bv[j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// dense^T x dense -> block-sparse.  One CTA: one 32x32 output block x one token chunk.
//   sparse_c[slot][c][r] = sum_t b[t, C*32+c] * a[t, R*32+r]
// grid = (nnz, splits); 64 threads, each a 4 (c) x 4 (r) register tile; splits > 1 accumulate
// with atomicAdd into a zero-filled output.
// ---------------------------------------------------------------------------------------------
template <bool kColMajor>
__device__ __forceinline__ void load_slab(float (*dst)[36], const float* __restrict__ src, int64_t ld,
                                          int64_t feat0, int64_t tok0, int64_t tok_end, int tid) {
    if (!kColMajor) {  // src[t * ld + f]
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = (tid >> 3) + 8 * i, f4 = (tid & 7) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tok0 + t < tok_end) v = *reinterpret_cast<const float4*>(src + (tok0 + t) * ld + feat0 + f4);
            *reinterpret_cast<float4*>(&dst[t][f4]) = v;
        }
    } else {  // src[f * ld + t]
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int e = tid + 64 * i, f = e >> 5, t = e & 31;
            dst[t][f] = (tok0 + t < tok_end) ? src[(feat0 + f) * ld + tok0 + t] : 0.f;
        }
    }
}

template <bool kAColMajor, bool kBColMajor>
__global__ void __launch_bounds__(64)
sddmm_simt_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t rows, int64_t cols,
                  int64_t tokens, float* __restrict__ sparse_c, const int2* __restrict__ blocks,
                  int64_t chunk_tokens, int use_atomics) {
    __shared__ __align__(16) float As[32][36];  // [token][r]
    __shared__ __align__(16) float Xs[32][36];  // [token][c]
    const int tid = threadIdx.x;
    const int tr = tid & 7, tc = tid >> 3;
    const int64_t slot = blockIdx.x;
    const int2 blk = blocks[slot];  // x: block-col C, y: block-row R
    const int64_t t_begin = (int64_t)blockIdx.y * chunk_tokens;
    const int64_t t_end = min(tokens, t_begin + chunk_tokens);
    const int64_t lda = kAColMajor ? tokens : rows;
    const int64_t ldb = kBColMajor ? tokens : cols;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int64_t t0 = t_begin; t0 < t_end; t0 += 32) {
        load_slab<kAColMajor>(As, a, lda, (int64_t)blk.y * 32, t0, t_end, tid);
        load_slab<kBColMajor>(Xs, b, ldb, (int64_t)blk.x * 32, t0, t_end, tid);
        __syncthreads();
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[t][tr * 4]);
            const float4 x4 = *reinterpret_cast<const float4*>(&Xs[t][tc * 4]);
            const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[i][0] = fmaf(xv[i], a4.x, acc[i][0]);
                acc[i][1] = fmaf(xv[i], a4.y, acc[i][1]);
                acc[i][2] = fmaf(xv[i], a4.z, acc[i][2]);
                acc[i][3] = fmaf(xv[i], a4.w, acc[i][3]);
            }
        }
        __syncthreads();
    }
    float* dst = sparse_c + slot * kBlockElems;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float* p = dst + (tc * 4 + i) * 32 + tr * 4;
        if (!use_atomics) {
            *reinterpret_cast<float4*>(p) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) atomicAdd(p + j, acc[i][j]);
        }
    }
}

__global__ void __launch_bounds__(256)
block_sumsq_kernel(const float* __restrict__ data, float* __restrict__ block_sumsq) {
    __shared__ float red[8];
    const int64_t slot = blockIdx.x;
    const float4 v = reinterpret_cast<const float4*>(data + slot * kBlockElems)[threadIdx.x];
    float s = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        block_sumsq[slot] = t;
    }
}

}  // namespace

cudaError_t launch_dsd_simt(const float* a, int64_t m, int64_t k, const int32_t* ptr, const int32_t* idx,
                            const float* data, int64_t n, float* out, const float* bias, bool dgrad,
                            bool out_colmajor, cudaStream_t stream) {
    if (m == 0 || n == 0) return cudaSuccess;
    const int64_t tiles = (m + 127) / 128;
    // grid.y is limited to 65535: walk the token range in slices of that many tiles
    for (int64_t t0 = 0; t0 < tiles; t0 += 65535) {
        const int64_t nt = tiles - t0 < 65535 ? tiles - t0 : 65535;
        const int64_t row0 = t0 * 128;
        const int64_t rows_here = (m - row0 < nt * 128) ? m - row0 : nt * 128;
        dim3 grid((unsigned)(n / 32), (unsigned)nt);
        const float* a_s = a + row0 * k;
        // column-major output of a slice needs the full leading dimension, so only one slice is allowed there
        if (out_colmajor && tiles > 65535) return cudaErrorInvalidValue;
        float* out_s = out_colmajor ? out : out + row0 * n;
        if (dgrad)
            dsd_simt_kernel<true><<<grid, 256, 0, stream>>>(a_s, rows_here, k, ptr, reinterpret_cast<const int2*>(idx),
                                                            data, n, out_s, bias, out_colmajor ? 1 : 0);
        else
            dsd_simt_kernel<false><<<grid, 256, 0, stream>>>(a_s, rows_here, k, ptr, reinterpret_cast<const int2*>(idx),
                                                             data, n, out_s, bias, out_colmajor ? 1 : 0);
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
}

cudaError_t launch_block_sumsq(const float* data, int64_t nnz, float* block_sumsq, cudaStream_t stream) {
    if (nnz == 0) return cudaSuccess;
    block_sumsq_kernel<<<(unsigned)nnz, 256, 0, stream>>>(data, block_sumsq);
    return cudaGetLastError();
}

cudaError_t launch_sddmm_simt(const float* a, bool a_colmajor, const float* b, bool b_colmajor, int64_t rows,
                              int64_t cols, int64_t tokens, float* sparse_c, const int32_t* blocks, int64_t nnz,
                              float* block_sumsq, cudaStream_t stream) {
    if (nnz == 0) return cudaSuccess;
    // enough CTAs to fill 148 SMs x 16 resident 64-thread CTAs, chunks of at least 256 tokens
    int64_t splits = (2368 + nnz - 1) / nnz;
    const int64_t max_splits = (tokens + 255) / 256;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    int64_t chunk = (tokens + splits - 1) / splits;
    chunk = (chunk + 31) / 32 * 32;
    if (chunk == 0) chunk = 32;
    splits = tokens > 0 ? (tokens + chunk - 1) / chunk : 1;
    const int use_atomics = splits > 1 ? 1 : 0;
    cudaError_t err;
    if (use_atomics) {
        err = cudaMemsetAsync(sparse_c, 0, (size_t)nnz * kBlockElems * sizeof(float), stream);
        if (err != cudaSuccess) return err;
    }
    dim3 grid((unsigned)nnz, (unsigned)splits);
    const int2* blk = reinterpret_cast<const int2*>(blocks);
#define BSMM_LAUNCH_SDDMM(AC, BC)                                                                              \
    sddmm_simt_kernel<AC, BC><<<grid, 64, 0, stream>>>(a, b, rows, cols, tokens, sparse_c, blk, chunk, use_atomics)
    if (a_colmajor) {
        if (b_colmajor) BSMM_LAUNCH_SDDMM(true, true);
        else BSMM_LAUNCH_SDDMM(true, false);
    } else {
        if (b_colmajor) BSMM_LAUNCH_SDDMM(false, true);
        else BSMM_LAUNCH_SDDMM(false, false);
    }
#undef BSMM_LAUNCH_SDDMM
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    if (block_sumsq != nullptr) return launch_block_sumsq(sparse_c, nnz, block_sumsq, stream);
    return cudaSuccess;
}

}  // namespace bsmm
