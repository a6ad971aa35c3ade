// Weight packing: turns the reference's `data` (slot s = 32x32 tile T[c][r] = W[R*32+r][C*32+c])
// into the shared-memory images the tcgen05 kernels fetch with one bulk copy per block, and
// produces the per-slot sum of squares behind block_norm in the same pass.
//
// Per slot and orientation the image is the B operand [mn][k] of a 128 x N x 32 UMMA step in the
// K-major, un-swizzled canonical layout (image32_offset / image16_offset):
//   fwd   (out = x * W^T): mn = r (output feature), k = c  -> value T[k][mn]
//   dgrad (out = dy * W ): mn = c (input feature),  k = r  -> value T[mn][k]
// The tf32 image interleaves hi = rna_tf32(w) and lo = rna_tf32(w - hi) per k-chunk, so that one
// N = 64 MMA reads [hi ; lo] and an N = 32 MMA reads hi alone.  Both parts are exact tf32 values:
// nothing depends on how the MMA unit would truncate fp32 bit patterns.  The bf16 hi | lo image
// (image16x3_offset) does the same with hi = bf16(w), lo = bf16(w - hi).
#include <cuda_bf16.h>

#include "bsmm_common.cuh"

namespace bsmm {
namespace {

__device__ __forceinline__ float tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// hi or lo part of the bf16 pair splitting: hi = bf16(w), lo = bf16(w - hi)
__device__ __forceinline__ float bf16_part(float w, uint32_t lo_part) {
    const float h = __bfloat162float(__float2bfloat16_rn(w));
    return lo_part ? w - h : h;   // (the caller rounds: hi is exact already)
}

// kMode: 0 = tf32 hi | lo images, 1 = bf16 images, 2 = bf16 hi | lo images
template <int kMode>
__global__ void __launch_bounds__(256)
pack_kernel(const float* __restrict__ data, int64_t nnz, uint8_t* __restrict__ packed,
            float* __restrict__ block_sumsq) {
    __shared__ float T[32][33];
    __shared__ float red[8];
    const int tid = threadIdx.x;
    const int64_t slot = blockIdx.x;

    const float4 v = reinterpret_cast<const float4*>(data + slot * kBlockElems)[tid];
    {
        const int c = tid >> 3, r4 = (tid & 7) * 4;
        T[c][r4 + 0] = v.x;
        T[c][r4 + 1] = v.y;
        T[c][r4 + 2] = v.z;
        T[c][r4 + 3] = v.w;
    }
    float s = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    if (tid == 0 && block_sumsq != nullptr) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        block_sumsq[slot] = t;
    }

    if (kMode == 0) {
        float* fwd = reinterpret_cast<float*>(packed + slot * (int64_t)kImage32Bytes);
        float* dgr = reinterpret_cast<float*>(packed + (nnz + slot) * (int64_t)kImage32Bytes);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w = tid + 256 * i;  // 32-bit word of the image: coalesced writes
            const uint32_t byte = w * 4;
            const uint32_t k = (byte / 1024u) * 4u + (byte % 16u) / 4u;
            const uint32_t lo_part = (byte % 1024u) / 512u;
            const uint32_t mn = ((byte % 512u) / 128u) * 8u + (byte % 128u) / 16u;
            const float wf = T[k][mn];
            const float hf = tf32_rna(wf);
            fwd[w] = lo_part ? tf32_rna(wf - hf) : hf;
            const float wd = T[mn][k];
            const float hd = tf32_rna(wd);
            dgr[w] = lo_part ? tf32_rna(wd - hd) : hd;
        }
    } else if (kMode == 2) {
        __nv_bfloat162* fwd = reinterpret_cast<__nv_bfloat162*>(packed + slot * (int64_t)kImage16x3Bytes);
        __nv_bfloat162* dgr = reinterpret_cast<__nv_bfloat162*>(packed + (nnz + slot) * (int64_t)kImage16x3Bytes);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = tid + 256 * i;  // 32-bit word = two consecutive k of one mn, hi or lo part
            const uint32_t byte = w * 4;
            const uint32_t k = (byte / 1024u) * 8u + (byte % 16u) / 2u;
            const uint32_t lo_part = (byte % 1024u) / 512u;
            const uint32_t mn = ((byte % 512u) / 128u) * 8u + (byte % 128u) / 16u;
            fwd[w] = __floats2bfloat162_rn(bf16_part(T[k][mn], lo_part), bf16_part(T[k + 1][mn], lo_part));
            dgr[w] = __floats2bfloat162_rn(bf16_part(T[mn][k], lo_part), bf16_part(T[mn][k + 1], lo_part));
        }
    } else {
        __nv_bfloat162* fwd = reinterpret_cast<__nv_bfloat162*>(packed + slot * (int64_t)kImage16Bytes);
        __nv_bfloat162* dgr = reinterpret_cast<__nv_bfloat162*>(packed + (nnz + slot) * (int64_t)kImage16Bytes);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t w = tid + 256 * i;  // 32-bit word = two consecutive k of one mn
            const uint32_t byte = w * 4;
            const uint32_t k = (byte / 512u) * 8u + (byte % 16u) / 2u;
            const uint32_t mn = ((byte % 512u) / 128u) * 8u + (byte % 128u) / 16u;
            fwd[w] = __floats2bfloat162_rn(T[k][mn], T[k + 1][mn]);
            dgr[w] = __floats2bfloat162_rn(T[mn][k], T[mn][k + 1]);
        }
    }
}

}  // namespace

cudaError_t launch_pack(const float* data, int64_t nnz, uint32_t precision, void* packed, float* block_sumsq,
                        cudaStream_t stream) {
    if (nnz == 0) return cudaSuccess;
    uint8_t* p = static_cast<uint8_t*>(packed);
    if (is_tf32_precision(precision))
        pack_kernel<0><<<(unsigned)nnz, 256, 0, stream>>>(data, nnz, p, block_sumsq);
    else if (precision == BSMM_PREC_BF16)
        pack_kernel<1><<<(unsigned)nnz, 256, 0, stream>>>(data, nnz, p, block_sumsq);
    else if (precision == BSMM_PREC_BF16X3)
        pack_kernel<2><<<(unsigned)nnz, 256, 0, stream>>>(data, nnz, p, block_sumsq);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace bsmm
