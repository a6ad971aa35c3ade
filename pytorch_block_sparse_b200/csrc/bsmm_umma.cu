// Tensor-core dense x block-sparse -> dense kernel for sm_100a (forward and dgrad of one
// block-sparse Linear; replaces the reference's cutlass::gemm::kernel<block_task>,
// cutlass/gemm/dispatch.h:185-218 and block_task.h:647-715).
//
// Tile: 128 tokens x G output block-rows (G*32 columns) per CTA.  The contraction axis is walked
// one 32-wide activation slab at a time, visiting only slabs for which the group has at least one
// block (the plan lists them, bsmm_plan.cu).
//
//   warp 0    producer : TMA tensor load of the [128 x 32] fp32 activation slab (128-B swizzle) and
//                        one 8 KiB linear bulk copy per block of its packed hi/lo weight images
//   warps 2-5 transform: slab smem -> registers, split into tf32 hi/lo, tcgen05.st into tensor
//                        memory (lane = token, column = k), which makes it the MMA's A operand
//   warp 1    MMA      : per block 4 k-steps x 3 passes (lo*hi, hi*lo, hi*hi) of
//                        tcgen05.mma kind::tf32 M=128 N=32 K=8, A from tensor memory, B from smem,
//                        accumulating the row's partial sum P[row] (32 fp32 columns of tensor memory)
//   warps 6-9 drain    : every kDrainEvery blocks of a row, tcgen05.ld P[row] and add it (fp32, round
//                        to nearest) to the row's master tile in shared memory; at the end the
//                        master tiles (initialised with the bias) leave through TMA tensor stores
//
// Why A from tensor memory: with both operands in shared memory an N=32 MMA re-reads 4 KiB of A per
// instruction and is bound by shared-memory bandwidth; from tensor memory only the 1 KiB weight
// image is read.  Why promotion: the tensor core's fp32 accumulate loses about 2e-8 (relative) per
// MMA, systematically, so a long row (96 blocks = 1152 MMAs) would exceed the 1e-5 error bound.
// Every mbarrier wait is bounded; on expiry the CTA raises the device status word and drains.
#include "bsmm_ptx.cuh"
#include "bsmm_umma.cuh"

namespace bsmm {

__device__ unsigned int g_device_status = 0;

namespace {

using namespace ptx;

constexpr int kTileTokens = 128;
constexpr uint32_t kXStageBytes = kTileTokens * 32 * 4;  // 16 KiB
constexpr uint32_t kWStageBytes = 2 * kImage32Bytes;     // 8 KiB: hi image, lo image
constexpr uint32_t kMasterBytes = kTileTokens * 32 * 4;  // 16 KiB per output block-row
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAStageCols = 64;                     // hi: 32 columns, lo: 32 columns
constexpr int kThreads = 320;

// Shared memory is split between the master tiles (G x 16 KiB) and the two load rings; tensor
// memory between the partial sums (G x 32 columns) and the split activation slabs.
template <int G>
struct Cfg {
    static constexpr int kXStages = 7 - G / 2;        // G=8: 3, 6: 4, 4: 5
    static constexpr int kWStages = 2 * kXStages;     // G=8: 6, 6: 8, 4: 10
    static constexpr int kAStages = 8 - G / 2;        // G=8: 4, 6: 5, 4: 6
    static constexpr uint32_t kAccCols = G * 32;
    static constexpr uint32_t kOffMaster = 0;
    static constexpr uint32_t kOffX = kOffMaster + G * kMasterBytes;
    static constexpr uint32_t kOffW = kOffX + kXStages * kXStageBytes;
    static constexpr uint32_t kOffBar = kOffW + kWStages * kWStageBytes;
    static constexpr int kNumBars = 2 * kXStages + 2 * kWStages + 2 * kAStages + 2 * G;
    static constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;  // + slack to align the base to 1 KiB
    static_assert(kAccCols + kAStages * kAStageCols <= kTmemCols, "tensor memory over-subscribed");
    static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");
};

struct DsdParams {
    const uint8_t* packed;     // image sets of this orientation, slot-major
    const int32_t* group_off;  // [groups + 1]
    const PlanEntry* entries;
    const float* bias;         // may be null
    float* out;
    unsigned int* status;      // device status word
    int64_t m, n;
    int32_t n_out_blocks, groups;
    int32_t out_colmajor;
    uint32_t x_bytes;          // bytes one activation-slab load delivers: min(128, m) rows of 128 B
};

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
dsd_umma_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_out,
                       const DsdParams p) {
    using C = Cfg<G>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t bar0 = smem_base + C::kOffBar;
    auto x_full = [&](int s) { return bar0 + 8u * s; };
    auto x_empty = [&](int s) { return bar0 + 8u * (C::kXStages + s); };
    auto w_full = [&](int s) { return bar0 + 8u * (2 * C::kXStages + s); };
    auto w_empty = [&](int s) { return bar0 + 8u * (2 * C::kXStages + C::kWStages + s); };
    auto a_full = [&](int s) { return bar0 + 8u * (2 * C::kXStages + 2 * C::kWStages + s); };
    auto a_empty = [&](int s) { return bar0 + 8u * (2 * C::kXStages + 2 * C::kWStages + C::kAStages + s); };
    auto p_ready = [&](int r) { return bar0 + 8u * (2 * C::kXStages + 2 * C::kWStages + 2 * C::kAStages + r); };
    auto p_taken = [&](int r) { return bar0 + 8u * (2 * C::kXStages + 2 * C::kWStages + 2 * C::kAStages + G + r); };
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kOffMisc);
    // misc[0]: tensor-memory base address, misc[1]: abort flag

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int g = blockIdx.x % p.groups;
    const int64_t tok0 = (int64_t)(blockIdx.x / p.groups) * kTileTokens;
    const int e0 = p.group_off[g], e1 = p.group_off[g + 1];
    const int nrows = min(G, p.n_out_blocks - g * G);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kXStages; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 128); }
        for (int s = 0; s < C::kWStages; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1); }
        for (int s = 0; s < C::kAStages; ++s) { mbar_init(a_full(s), 128); mbar_init(a_empty(s), 1); }
        for (int r = 0; r < G; ++r) { mbar_init(p_ready(r), 1); mbar_init(p_taken(r), 128); }
        misc[1] = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_base + C::kOffMisc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    volatile uint32_t* abort_flag = &misc[1];

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int xs = 0, ws = 0;
            uint32_t xph = 0, wph = 0;
            for (int e = e0; e < e1; ++e) {
                const PlanEntry ent = p.entries[e];
                if (ent.flags & kPlanFirst) {
                    if (!mbar_wait(x_empty(xs), xph ^ 1u, abort_flag)) break;
                    mbar_arrive_expect_tx(x_full(xs), p.x_bytes);
                    tma_load_2d(smem_base + C::kOffX + xs * kXStageBytes, &tmap_a, ent.inner * 32, (int32_t)tok0,
                                x_full(xs));
                    if (++xs == C::kXStages) { xs = 0; xph ^= 1u; }
                }
                if (!mbar_wait(w_empty(ws), wph ^ 1u, abort_flag)) break;
                mbar_arrive_expect_tx(w_full(ws), kWStageBytes);
                bulk_load(smem_base + C::kOffW + ws * kWStageBytes, p.packed + (int64_t)ent.slot * kWStageBytes,
                          kWStageBytes, w_full(ws));
                if (++ws == C::kWStages) { ws = 0; wph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(2u, 128u, 32u, false, false);
            int ws = 0, as = 0;
            uint32_t wph = 0, aph = 0;
            uint32_t started = 0;   // bit r: P[r] holds a partial sum of the current segment
            uint32_t pending = 0;   // bit r: a promotion of P[r] was requested and not yet seen taken
            uint32_t taken_ph = 0;  // bit r: parity of the next p_taken[r] phase to wait for
            uint32_t a_hi = 0;
            for (int e = e0; e < e1; ++e) {
                const PlanEntry ent = p.entries[e];
                const uint32_t rbit = 1u << ent.row;
                if (ent.flags & kPlanFirst) {
                    if (!mbar_wait(a_full(as), aph, abort_flag)) break;
                    a_hi = tmem + C::kAccCols + as * kAStageCols;
                }
                if (!mbar_wait(w_full(ws), wph, abort_flag)) break;
                if (pending & rbit) {  // the drain warps must have read P[row] before it is overwritten
                    if (!mbar_wait(p_taken(ent.row), (taken_ph >> ent.row) & 1u, abort_flag)) break;
                    taken_ph ^= rbit;
                    pending &= ~rbit;
                }
                tc_fence_after();
                const uint32_t w_addr = smem_base + C::kOffW + ws * kWStageBytes;
                const uint64_t b_hi = smem_desc_noswizzle(w_addr, 512, 128);
                const uint64_t b_lo = smem_desc_noswizzle(w_addr + kImage32Bytes, 512, 128);
                const uint32_t d = tmem + ent.row * 32;
                uint32_t accumulate = (started & rbit) ? 1u : 0u;
                started |= rbit;
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint64_t koff = (uint64_t)((s * 1024) >> 4);  // two 512-B k-chunks per step
                    mma_ts_tf32(d, a_hi + 32 + s * 8, b_hi + koff, idesc, accumulate);  // lo * hi
                    mma_ts_tf32(d, a_hi + s * 8, b_lo + koff, idesc, 1u);               // hi * lo
                    mma_ts_tf32(d, a_hi + s * 8, b_hi + koff, idesc, 1u);               // hi * hi
                    accumulate = 1u;
                }
                mma_commit(w_empty(ws));
                if (++ws == C::kWStages) { ws = 0; wph ^= 1u; }
                if (ent.flags & kPlanLast) {
                    mma_commit(a_empty(as));
                    if (++as == C::kAStages) { as = 0; aph ^= 1u; }
                }
                if (ent.flags & kPlanDrain) {
                    mma_commit(p_ready(ent.row));
                    pending |= rbit;
                    started &= ~rbit;
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ transform
        const int quarter = warp & 3;              // tensor-memory lane quarter this warp may access
        const int row = quarter * 32 + lane;       // token inside the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        int xs = 0, as = 0;
        uint32_t xph = 0, aph = 0;
        for (int e = e0; e < e1; ++e) {
            const int flags = p.entries[e].flags;
            if (!(flags & kPlanFirst)) continue;
            if (!__all_sync(0xffffffffu, mbar_wait(x_full(xs), xph, abort_flag))) break;
            uint32_t hi[32], lo[32];
            {
                const uint8_t* xrow = smem_gen + C::kOffX + xs * kXStageBytes + row * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // 128-B swizzle: the 16-B chunk index is XORed with (row mod 8)
                    const float4 v = *reinterpret_cast<const float4*>(xrow + ((j ^ (row & 7)) << 4));
                    const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t h = tf32_rna_bits(f[q]);
                        hi[j * 4 + q] = h;
                        lo[j * 4 + q] = tf32_rna_bits(f[q] - __uint_as_float(h));
                    }
                }
            }
            mbar_arrive(x_empty(xs));
            if (++xs == C::kXStages) { xs = 0; xph ^= 1u; }
            if (!__all_sync(0xffffffffu, mbar_wait(a_empty(as), aph ^ 1u, abort_flag))) break;
            tc_fence_after();
            const uint32_t a_hi = tmem_lane + C::kAccCols + as * kAStageCols;
            tmem_st32(a_hi, hi);
            tmem_st32(a_hi + 32, lo);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(a_full(as));
            if (++as == C::kAStages) { as = 0; aph ^= 1u; }
        }
    } else {
        // ------------------------------------------------------------------ drain + epilogue
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t tmem_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        // this thread's 128-B row of master tile r is at master + r * kMasterBytes, its 16-B chunks
        // swizzled like TMA's 128-B mode so that the tile can leave through a tensor store
        uint8_t* master = smem_gen + C::kOffMaster + row * 128;
        const int swz = row & 7;

        // master tiles start as the bias (or zero): rows without any block come out right by themselves
        for (int r = 0; r < nrows; ++r) {
            const float* brow = p.bias != nullptr ? p.bias + ((int64_t)g * G + r) * 32 : nullptr;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                if (brow != nullptr) b = __ldg(reinterpret_cast<const float4*>(brow) + j);
                *reinterpret_cast<float4*>(master + r * kMasterBytes + ((j ^ swz) << 4)) = b;
            }
        }

        uint32_t ready_ph = 0;  // bit r: parity of the next p_ready[r] phase
        bool ok = true;
        for (int e = e0; e < e1; ++e) {
            const PlanEntry ent = p.entries[e];
            if (!(ent.flags & kPlanDrain)) continue;
            const int r = ent.row;
            ok = __all_sync(0xffffffffu, mbar_wait(p_ready(r), (ready_ph >> r) & 1u, abort_flag));
            if (!ok) break;
            ready_ph ^= 1u << r;
            tc_fence_after();
            uint32_t acc[32];
            tmem_ld32(tmem_lane + r * 32, acc);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(p_taken(r));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float4* mp = reinterpret_cast<float4*>(master + r * kMasterBytes + ((j ^ swz) << 4));
                float4 v = *mp;
                v.x += __uint_as_float(acc[j * 4 + 0]);
                v.y += __uint_as_float(acc[j * 4 + 1]);
                v.z += __uint_as_float(acc[j * 4 + 2]);
                v.w += __uint_as_float(acc[j * 4 + 3]);
                *mp = v;
            }
        }

        // every drain warp reaches this barrier, also after giving up on a wait (its loop above is bounded)
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok && *abort_flag == 0) {
            if (!p.out_colmajor) {
                // master tiles -> global through TMA tensor stores (rows beyond m are clipped by the map)
                if (warp == 6 && lane == 0) {
                    for (int r = 0; r < nrows; ++r)
                        tma_store_2d(&tmap_out, smem_base + C::kOffMaster + r * kMasterBytes,
                                     (int32_t)(((int64_t)g * G + r) * 32), (int32_t)tok0);
                    bulk_commit_group();
                    bulk_wait_group<0>();
                }
            } else {
                const int64_t tok = tok0 + row;
                if (tok < p.m) {
                    for (int r = 0; r < nrows; ++r) {
                        const int64_t col0 = ((int64_t)g * G + r) * 32;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 v =
                                *reinterpret_cast<const float4*>(master + r * kMasterBytes + ((j ^ swz) << 4));
                            p.out[(col0 + j * 4 + 0) * p.m + tok] = v.x;
                            p.out[(col0 + j * 4 + 1) * p.m + tok] = v.y;
                            p.out[(col0 + j * 4 + 2) * p.m + tok] = v.z;
                            p.out[(col0 + j * 4 + 3) * p.m + tok] = v.w;
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicOr(p.status, 1u);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// cuTensorMapEncodeTiled, resolved at run time so the library needs no link-time libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

template <int G>
cudaError_t launch_dsd_g(const CUtensorMap& tmap_a, const CUtensorMap& tmap_out, const DsdParams& p, int64_t tiles,
                         cudaStream_t stream) {
    // per call: the attribute is per device and the caller may switch devices
    cudaError_t err = cudaFuncSetAttribute(dsd_umma_tf32x3_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)Cfg<G>::kSmemBytes);
    if (err != cudaSuccess) return err;
    dsd_umma_tf32x3_kernel<G>
        <<<(unsigned)(p.groups * tiles), kThreads, Cfg<G>::kSmemBytes, stream>>>(tmap_a, tmap_out, p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                         uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * elem_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t device_status_address(unsigned int** addr) {
    constexpr int kMaxDevices = 64;
    static unsigned int* cache[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_device_status);
        if (err != cudaSuccess) return err;
        cache[dev] = static_cast<unsigned int*>(p);
    }
    *addr = cache[dev];
    return cudaSuccess;
}

cudaError_t launch_dsd_umma(const void* a, int64_t m, int64_t k, int64_t nnz, const void* packed, const void* plan,
                            int group, int64_t n, void* out, const float* bias, uint32_t precision, bool dgrad,
                            bool out_colmajor, cudaStream_t stream) {
    if (precision != BSMM_PREC_TF32X3) return cudaErrorNotSupported;
    if (!plan_group_valid(group)) return cudaErrorInvalidValue;
    if (m == 0 || n == 0) return cudaSuccess;
    if (k == 0) return cudaErrorInvalidValue;  // nothing to contract over; a tensor map cannot describe it
    const int64_t n_out_blocks = n / 32;
    const int64_t groups = plan_groups(n_out_blocks, group);
    const int64_t tiles = (m + kTileTokens - 1) / kTileTokens;
    if (groups * tiles > 0x7fffffffll || m > 0x7fffffffll) return cudaErrorInvalidValue;

    // The boxes never exceed the tensors: with fewer than 128 tokens the slab load fills only the
    // first m rows; the remaining tensor-memory lanes hold stale values whose outputs are never stored.
    const uint32_t box_rows = (uint32_t)(m < kTileTokens ? m : kTileTokens);
    CUtensorMap tmap_a, tmap_out;
    cudaError_t err = make_tmap_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a, (uint64_t)k, (uint64_t)m, 32,
                                   box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess) return err;
    if (!out_colmajor) {
        err = make_tmap_2d(&tmap_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, out, (uint64_t)n, (uint64_t)m, 32, box_rows,
                           CU_TENSOR_MAP_SWIZZLE_128B);
        if (err != cudaSuccess) return err;
    } else {
        tmap_out = tmap_a;  // unused by the kernel in this mode
    }

    DsdParams p;
    const int64_t slot_bytes = packed_slot_bytes(BSMM_PREC_TF32X3);
    p.packed = static_cast<const uint8_t*>(packed) + (dgrad ? nnz * slot_bytes : 0);
    p.group_off = static_cast<const int32_t*>(plan);
    p.entries = reinterpret_cast<const PlanEntry*>(static_cast<const uint8_t*>(plan) +
                                                   plan_entries_offset(n_out_blocks, group));
    p.bias = bias;
    p.out = static_cast<float*>(out);
    err = device_status_address(&p.status);
    if (err != cudaSuccess) return err;
    p.m = m;
    p.n = n;
    p.n_out_blocks = (int32_t)n_out_blocks;
    p.groups = (int32_t)groups;
    p.out_colmajor = out_colmajor ? 1 : 0;
    p.x_bytes = box_rows * 128u;
    switch (group) {
        case 4: return launch_dsd_g<4>(tmap_a, tmap_out, p, tiles, stream);
        case 6: return launch_dsd_g<6>(tmap_a, tmap_out, p, tiles, stream);
        default: return launch_dsd_g<8>(tmap_a, tmap_out, p, tiles, stream);
    }
}

cudaError_t read_device_status(unsigned int* status, bool clear) {
    cudaError_t err = cudaMemcpyFromSymbol(status, g_device_status, sizeof(unsigned int));
    if (err != cudaSuccess) return err;
    if (clear && *status != 0) {
        const unsigned int zero = 0;
        err = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(unsigned int));
    }
    return err;
}

int64_t sddmm_umma_workspace_bytes(int64_t, int64_t, int64_t, int64_t, uint32_t) { return 0; }

cudaError_t launch_sddmm_umma(const void*, const void*, int64_t, int64_t, int64_t, float*, const int32_t*, int64_t,
                              float*, void*, uint32_t, cudaStream_t) {
    return cudaErrorNotSupported;
}

}  // namespace bsmm
