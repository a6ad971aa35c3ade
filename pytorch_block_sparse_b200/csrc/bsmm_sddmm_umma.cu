// Tensor-core dense^T x dense -> block-sparse kernel (the wgrad of one block-sparse Linear) for
// sm_100a; replaces the reference's cutlass::gemm::kernel<block_task_back>
// (cutlass/gemm/dispatch_back.h:186-218, block_task_back.h:643-707).
//
//   out[slot][c][r] = sum over tokens t of X[t, C*32 + c] * dY[t, R*32 + r]
//
// A CTA owns one "item": up to 8 blocks of ONE block-row R (a CSR row segment) and one range of
// tokens.  Four blocks of the row form a chunk and fill the 128 rows of one MMA:
//   D[128 = 4 blocks x 32 c, 32 = r] += A[128 x K] * B[32 x K]^T,   K = tokens, 8 per instruction.
// D is already the block's storage layout (row c holds 32 consecutive r).  A "unit" is one chunk times one
// 32-token step: 8 MMAs.
//
// B = the dY slab of row R, token-major in memory, i.e. MN-major for the MMA: a TMA box of 32 tokens x 32
// features with the 128-byte / 32-byte-atom swizzle IS the canonical MN-major tf32 operand tile, read from
// shared memory where TMA put it.  A = the chunk's four X slabs, which the split warps carry through
// registers into tensor memory, transposed (lane = feature, column = token) and split into hi | lo: reading
// A from shared memory as well made the kernel shared-memory-bandwidth bound (92 KB per unit).
//
//   warps 0-1   X producers : TMA, four X slabs per unit (units by parity)
//   warp 2      dY producer : TMA, one dY slab per step
//   warps 3-4   dY split    : lo = v - trunc_tf32(v) of the dY slab (half each) into a second tile of the same layout
//                             (the tensor core reads only the tf32 bits of an operand, so the raw slab is hi)
//   warps 5-6   MMA         : warp c owns chunk c (two chunks per item): per unit and k-step (8 tokens)
//                             x x [dy ; dy_lo] (N = 64) and x_lo x dy (N = 32), tcgen05.mma kind::tf32, M = 128,
//                             into the main | correction columns of the chunk
//   warps 7-18  X split     : three groups of four (unit mod 3): shared memory -> registers (transposing
//                             reads, conflict-free under the 128-byte swizzle) -> hi, lo -> tensor memory;
//                             six stages, so a chunk's copies run up to three steps ahead of its MMAs
//   warps 19-22 drain       : every 1024 tokens tcgen05.ld each chunk's columns and add main + correction
//                             (fp32, round to nearest) to the chunk's master tile in shared memory; final
//                             store of the master tiles to global
//
// The promotion bounds the tensor core's systematic accumulate error (about 2e-8 relative per MMA).
// Token ranges (grid.y > 1) write partial results to the workspace; a second kernel sums them in a
// fixed order (deterministic, no atomics) and produces the per-slot sum of squares.
#include <cuda_bf16.h>

#include "bsmm_ptx.cuh"
#include "bsmm_umma.cuh"

namespace bsmm {
namespace {

using namespace ptx;

constexpr int kChunks = 2;                 // chunks (of 4 blocks) per item
constexpr int kItemBlocks = 4 * kChunks;   // 8
constexpr int kStepTokens = 32;
constexpr int kDrainSteps = 32;            // promote every 1024 tokens: 128 accumulations of the main term
constexpr uint32_t kSlabBytes = 32 * 32 * 4;            // 4 KiB: [32 tokens][32 features], 128-byte rows
constexpr uint32_t kKStepBytes = 8 * 128;               // one MMA k-step = 8 token rows
constexpr uint32_t kXStageBytes = 4 * kSlabBytes;       // one unit's four X slabs
constexpr uint32_t kDyStageBytes = 2 * kSlabBytes;      // raw slab | its lo part
constexpr uint32_t kMasterBytes = 128 * 32 * 4;         // 16 KiB per chunk
constexpr int kStages = 6;                              // X stages in shared memory = A stages in tensor memory:
                                                        // three per chunk, so a chunk's copy runs ahead of its MMAs
constexpr int kDyStages = 4;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kChunkCols = 64;                     // main | correction
constexpr uint32_t kAccCols = kChunks * kChunkCols;     // 128
constexpr uint32_t kAStageCols = 64;                    // x_hi | x_lo, 32 tokens each
constexpr int kXProducers = 2, kDyProducerWarp = 2, kDySplitWarp = 3, kDySplitWarps = 2;  // halves of the slab
constexpr int kFirstMmaWarp = kDySplitWarp + kDySplitWarps;
constexpr int kSplitGroups = 3;  // groups of four split warps; unit u goes to group u mod kSplitGroups
constexpr int kFirstSplitWarp = kFirstMmaWarp + kChunks, kSplitWarps = 4 * kSplitGroups;
constexpr int kFirstDrainWarp = kFirstSplitWarp + kSplitWarps;
constexpr int kThreads = 32 * (kFirstDrainWarp + 4);

constexpr uint32_t kOffMaster = 0;
constexpr uint32_t kOffX = kOffMaster + kChunks * kMasterBytes;
constexpr uint32_t kOffDy = kOffX + kStages * kXStageBytes;
constexpr uint32_t kOffBar = kOffDy + kDyStages * kDyStageBytes;
constexpr int kNumBars = 3 * kStages + 3 * kDyStages + 2 * kChunks;
constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffMisc + 32 + 1024;
static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");
static_assert(kAccCols + kStages * kAStageCols <= kTmemCols, "tensor memory over-subscribed");
static_assert(kStages % kXProducers == 0 && kStages % kSplitGroups == 0,
              "a stage must stay with one producer warp and one split-warp group");

// Item table: [0] = item count; item i at int32 offsets 4 + 4*i: {block-row, first CSR entry, blocks, 0}
struct SddmmParams {
    const int32_t* items;
    const int2* idx;       // CSR entries: (block-col, slot)
    float* out;            // sparse_c, or the workspace when the token axis is split
    float* block_sumsq;    // may be null; only written when the token axis is not split
    unsigned int* status;
    int64_t tokens;
    int64_t tokens_per_split;  // multiple of kStepTokens
    int64_t split_stride;      // floats between two splits' partial results
};

// MN-major tf32 operand made of swizzle atoms of 4 k-rows x 128 bytes of the M/N axis (128-byte swizzle
// with 32-byte atomicity): atoms along M/N are `atom_stride` bytes apart (leading byte offset), the
// 4-row groups along K follow each other at 512 bytes (stride byte offset).
__device__ __forceinline__ uint64_t smem_desc_mnmajor_sw128(uint32_t addr, uint32_t atom_stride) {
    return smem_desc_sw128_base32(addr, atom_stride, 512);
}

// kPasses = 3: 3xTF32 as described above; kPasses = 1: single-pass TF32 (no lo parts, no correction columns);
// kPasses = 0: bf16 operands (kind::f16, K = 16 per instruction): the dY split warp writes the slab transposed
// and rounded as a K-major bf16 tile (the layout of the bf16 weight images), the X split warps pack token pairs
// kPasses = 4: bf16 operands that are bf16 tensors in memory already (token-major): the dY box, loaded with the
// 64-byte swizzle, IS the MN-major canonical bf16 operand tile (atoms of 8 token rows x 64 bytes), so the dY split
// warps have nothing to do; the X split warps read 2-byte values and pack token pairs.
// kPasses = 5: three products of bf16 hi and lo parts of fp32 tensors (token-major), fp32-class accuracy with half the
// instructions of 3xTF32: the dY split warps write hi = bf16(v) and lo = bf16(v - hi) as two MN-major bf16 tiles
// (the 64-byte-swizzle layout of the bf16-tensor mode; [hi ; lo] is the N = 64 operand), the X split warps pack
// token pairs of hi and of lo.
// kXFm / kDyFm: the operand is given feature-major ([features, tokens] contiguous, the reference's other
// contiguity case, native/block_sparse_cutlass_kernel_back.cu:145-157) instead of token-major.  The TMA box is then
// 32 features x 32 tokens with 128-byte token rows: for X that is already the orientation tensor memory wants
// (lane = feature), read with 16-byte loads instead of the transposing 4-byte ones; for dY it is the K-major
// canonical operand tile (plain 128-byte swizzle, 8-feature atoms of 1 KiB).
template <int kPasses, bool kXFm, bool kDyFm>
__global__ void __launch_bounds__(kThreads, 1)
sddmm_umma_tf32_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_dy,
                         const SddmmParams p) {
    constexpr bool kBf16 = kPasses == 0 || kPasses == 4 || kPasses == 5, kIo16 = kPasses == 4;
    constexpr bool kSplit = kPasses == 3 || kPasses == 5;   // hi and lo parts, correction columns
    static_assert((!kIo16 && kPasses != 5) || (!kXFm && !kDyFm), "bf16 tensors and the bf16 hi | lo mode take token-major operands");
    constexpr uint32_t kLoadSlabBytes = kIo16 ? kSlabBytes / 2 : kSlabBytes;   // what one TMA box delivers
    const int n_items = p.items[0];
    if ((int)blockIdx.x >= n_items) return;
    const int4 item = reinterpret_cast<const int4*>(p.items + 4)[blockIdx.x];
    const int brow = item.x, ent0 = item.y, nblk = item.z;
    const int nchunks = (nblk + 3) >> 2;
    const int64_t t_begin = (int64_t)blockIdx.y * p.tokens_per_split;
    const int64_t t_end = min(p.tokens, t_begin + p.tokens_per_split);
    const int nsteps = (int)((t_end - t_begin + kStepTokens - 1) / kStepTokens);
    const int nunits = nsteps * nchunks;  // unit u = step * nchunks + chunk uses stage u mod kStages

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + kOffBar;
    auto x_full = [&](int s) { return bar0 + 8u * s; };                      // TMA delivered the unit's slabs
    auto x_empty = [&](int s) { return bar0 + 8u * (kStages + s); };         // the split warps have read them
    auto a_empty = [&](int s) { return bar0 + 8u * (2 * kStages + s); };     // the MMAs reading the tensor-memory stage completed
    auto dy_full = [&](int s) { return bar0 + 8u * (3 * kStages + s); };
    auto dylo_full = [&](int s) { return bar0 + 8u * (3 * kStages + kDyStages + s); };
    auto dy_empty = [&](int s) { return bar0 + 8u * (3 * kStages + 2 * kDyStages + s); };
    auto p_ready = [&](int c) { return bar0 + 8u * (3 * kStages + 3 * kDyStages + c); };
    auto p_taken = [&](int c) { return bar0 + 8u * (3 * kStages + 3 * kDyStages + kChunks + c); };
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + kOffMisc);
    // misc[0]: tensor-memory base address, misc[1]: abort flag, misc[2 + stage]: how many split warps have
    // completed a copy into that tensor-memory stage so far -- its u-th unit may be read at 4 * (u + 1)
    auto a_count = [&](int s) { return smem_base + kOffMisc + 8u + 4u * s; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 128); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < kDyStages; ++s) { mbar_init(dy_full(s), 1); mbar_init(dylo_full(s), 32 * kDySplitWarps); mbar_init(dy_empty(s), nchunks); }
        for (int c = 0; c < kChunks; ++c) { mbar_init(p_ready(c), 1); mbar_init(p_taken(c), 128); }
        misc[1] = 0;
        for (int s = 0; s < kStages; ++s) misc[2 + s] = 0;
        fence_mbar_init();
    }
    if (warp == kFirstMmaWarp) {
        tmem_alloc(smem_base + kOffMisc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    volatile uint32_t* abort_flag = &misc[1];

    // Waits do not branch on their result in the common case (a conditional branch costs a lone warp ~40
    // cycles).  A wait that gives up (bounded, see mbar_wait) sets `bad`; the issuing instructions are
    // predicated on it and the role loops test it once per iteration.
    uint32_t bad = 0;
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (!mbar_try_wait(bar, parity) && !mbar_wait(bar, parity, abort_flag)) bad = 1;
    };
    auto wait_count = [&](uint32_t addr, uint32_t target) {  // bounded like mbar_wait
        if ((int32_t)(smem_load_acquire(addr) - target) < 0) {
            const long long t0 = clock64();
            for (;;) {
                if ((int32_t)(smem_load_acquire(addr) - target) >= 0) break;
                if (*abort_flag != 0) { bad = 1; break; }
                if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; bad = 1; break; }
            }
        }
    };

    // the item's CSR entries, one per lane (at most 16), handed out by shuffle
    const int2 my_ent = lane < nblk ? __ldg(p.idx + ent0 + lane) : make_int2(0, 0);

    // a step is a promotion point when it closes a 1024-token segment or the token range
    auto drain_step = [&](int step) { return ((step + 1) % kDrainSteps) == 0 || step + 1 == nsteps; };

    if (warp < kXProducers) {
        // ------------------------------------------------------------------ X producers
        // Warp w loads the units of parity w.  With two chunks that is chunk w of every step, with one chunk
        // every other step; either way the unit number grows by two per iteration.  The block columns of both
        // chunks are fetched from the lanes once, so the loop has no shuffles and no index loops.
        static_assert(kChunks == 2 && kXProducers == 2, "unit parity = producer warp");
        const int ch = nchunks == 2 ? warp : 0;
        const int nb = min(4, nblk - ch * 4);
        int bcol[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) bcol[j] = __shfl_sync(0xffffffffu, my_ent.x, ch * 4 + j) * 32;
        int xs = warp;            // stage of unit u: u mod kStages, kept incrementally
        uint32_t parity = 1u;     // of the stage's release barrier: (u / kStages) & 1, inverted
        const int step_stride = nchunks == 2 ? 1 : 2;
        for (int step = nchunks == 2 ? 0 : warp; step < nsteps; step += step_stride) {
            const int32_t tok = (int32_t)(t_begin + (int64_t)step * kStepTokens);
            wait(x_empty(xs), parity);
            const uint32_t dst = smem_base + kOffX + xs * kXStageBytes;
            if (elect_one() & (bad == 0)) {
                mbar_arrive_expect_tx(x_full(xs), nb * kLoadSlabBytes);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (j < nb) {
                        if (kXFm) tma_load_2d(dst + j * kSlabBytes, &tmap_x, tok, bcol[j], x_full(xs));
                        else tma_load_2d(dst + j * kSlabBytes, &tmap_x, bcol[j], tok, x_full(xs));
                    }
            }
            const bool wrap = xs + 2 >= kStages;
            xs = wrap ? xs + 2 - kStages : xs + 2;
            parity ^= wrap ? 1u : 0u;
        }
    } else if (warp == kDyProducerWarp) {
        // ------------------------------------------------------------------ dY producer
        for (int step = 0; step < nsteps && !bad; ++step) {
            const int ds = step & (kDyStages - 1);
            const int32_t tok = (int32_t)(t_begin + (int64_t)step * kStepTokens);
            wait(dy_empty(ds), ((uint32_t)(step / kDyStages) & 1u) ^ 1u);
            if (elect_one() && !bad) {
                mbar_arrive_expect_tx(dy_full(ds), kLoadSlabBytes);
                if (kDyFm) tma_load_2d(smem_base + kOffDy + ds * kDyStageBytes, &tmap_dy, tok, brow * 32, dy_full(ds));
                else tma_load_2d(smem_base + kOffDy + ds * kDyStageBytes, &tmap_dy, brow * 32, tok, dy_full(ds));
            }
        }
    } else if (warp < kFirstMmaWarp) {
        // ------------------------------------------------------------------ dY split
        // lo = v - trunc_tf32(v), elementwise at the same offset of the stage's second half: the swizzle
        // needs no decoding; consecutive lanes take consecutive 16-byte chunks
        const int half = warp - kDySplitWarp;  // which half of the slab this warp converts
        for (int step = 0; step < nsteps && kPasses != 1 && !kIo16; ++step) {
            const int ds = step & (kDyStages - 1);
            wait(dy_full(ds), (uint32_t)(step / kDyStages) & 1u);
            if (__any_sync(0xffffffffu, bad != 0)) break;
            uint8_t* base = smem_gen + kOffDy + ds * kDyStageBytes;
            if (kPasses == 5) {
                // this warp's 16 tokens x 4 groups of 8 features, two per lane.  The raw slab lies under the plain
                // 128-byte swizzle (16-byte chunk index XOR token mod 8); the bf16 tiles have 64-byte token rows under
                // the 64-byte swizzle (chunk index XOR (token / 2) mod 4): hi at +4 KiB, lo at +6 KiB.
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int u = lane + 32 * i;
                    const int t = 16 * half + (u >> 2), g = u & 3;
                    const float4 v0 = *reinterpret_cast<const float4*>(base + t * 128 + (((2 * g) ^ (t & 7)) << 4));
                    const float4 v1 = *reinterpret_cast<const float4*>(base + t * 128 + (((2 * g + 1) ^ (t & 7)) << 4));
                    const float f[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    uint32_t h[4], l[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) split_bf16x2(f[2 * q], f[2 * q + 1], h[q], l[q]);
                    const uint32_t off = (uint32_t)(t * 64 + ((g ^ ((t >> 1) & 3)) << 4));
                    *reinterpret_cast<uint4*>(base + kSlabBytes + off) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(base + kSlabBytes + kSlabBytes / 2 + off) = make_uint4(l[0], l[1], l[2], l[3]);
                }
            } else if (kPasses == 3) {
#pragma unroll
                for (int i = 4 * half; i < 4 * half + 4; ++i) {
                    const float4 v = *reinterpret_cast<const float4*>(base + (lane + 32 * i) * 16);
                    float4 l;
                    l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
                    l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
                    l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
                    l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
                    *reinterpret_cast<float4*>(base + kSlabBytes + (lane + 32 * i) * 16) = l;
                }
            } else if (kDyFm) {
                // lane = feature r owns row r of the slab: 32 tokens = 8 chunks of 16 bytes (chunk index XOR r mod 8)
                const uint8_t* rowp = base + lane * 128;
#pragma unroll
                for (int j = 2 * half; j < 2 * half + 2; ++j) {   // this warp's 16 tokens: chunks 4 half .. 4 half + 3
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int c = 2 * j + q;
                        const float4 v = *reinterpret_cast<const float4*>(rowp + ((c ^ (lane & 7)) << 4));
                        const __nv_bfloat162 p01 = __floats2bfloat162_rn(v.x, v.y), p23 = __floats2bfloat162_rn(v.z, v.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<const uint32_t*>(&p01);
                        packed.y = *reinterpret_cast<const uint32_t*>(&p23);
                        // tokens 4c .. 4c + 3 of feature r: 8 consecutive bytes of the K-major bf16 tile
                        *reinterpret_cast<uint2*>(base + kSlabBytes + image16_offset((uint32_t)lane, (uint32_t)(4 * c))) = packed;
                    }
                }
            } else {
                // lane = feature r; the slab (plain 128-byte swizzle in this mode) is read along the tokens
                // and written eight tokens (one 16-byte core-matrix row) at a time: consecutive lanes, consecutive rows
                const uint8_t* col = base + ((lane & 3) << 2);
#pragma unroll
                for (int t0 = 16 * half; t0 < 16 * half + 16; t0 += 8) {
                    uint32_t pk[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int t = t0 + 2 * i;   // (t0 is a multiple of 8: t mod 8 = 2 i)
                        const float v0 = *reinterpret_cast<const float*>(col + t * 128 + (((lane >> 2) ^ (2 * i)) << 4));
                        const float v1 = *reinterpret_cast<const float*>(col + (t + 1) * 128 + (((lane >> 2) ^ (2 * i + 1)) << 4));
                        const __nv_bfloat162 pr = __floats2bfloat162_rn(v0, v1);  // k = t low half, k = t + 1 high half
                        pk[i] = *reinterpret_cast<const uint32_t*>(&pr);
                    }
                    *reinterpret_cast<uint4*>(base + kSlabBytes + image16_offset((uint32_t)lane, (uint32_t)t0)) =
                        make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            fence_proxy_async_smem();  // generic-proxy writes, read by the MMA through the async proxy
            mbar_arrive(dylo_full(ds));
        }
    } else if (warp < kFirstSplitWarp) {
        // ------------------------------------------------------------------ MMA issuers
        const int ch = warp - kFirstMmaWarp;  // accumulations into one chunk stay in one thread's program order
        constexpr uint32_t idesc_wide = make_idesc(2u, 128u, 64u, false, !kDyFm);
        constexpr uint32_t idesc_narrow = make_idesc(2u, 128u, 32u, false, !kDyFm);
        constexpr uint32_t idesc_bf16 = make_idesc(1u, 128u, 32u, false, kIo16 || kPasses == 5);  // bf16 tensors, hi | lo tiles: B is MN-major
        constexpr uint32_t idesc_bf16_wide = make_idesc(1u, 128u, 64u, false, true);
        // The loop is cut into promotion segments (kDrainSteps steps) so that the per-step body has no
        // first-step / last-step decisions: a conditional branch costs this lone warp ~40 cycles, and the
        // body's length bounds how fast a chunk's stages turn around.
        uint32_t taken_ph = 0;
        int as = ch;               // stage of unit u = step * nchunks + ch: u mod kStages, kept incrementally
        uint32_t a_target = 4;     // 4 * (u / kStages + 1): the stage's copy count that means "unit u is there"
        const uint32_t d = tmem + ch * kChunkCols;
        const uint32_t p_bar = p_ready(ch);
        for (int seg = 0; seg < nsteps && ch < nchunks; seg += kDrainSteps) {
            const int seg_end = min(nsteps, seg + kDrainSteps);
            if (seg != 0) {  // the drain warps must have read the columns before the segment's first MMA overwrites them
                wait(p_taken(ch), taken_ph);
                taken_ph ^= 1u;
            }
            uint32_t acc0 = 0u;  // the segment's first MMA overwrites the columns
            for (int step = seg; step < seg_end; ++step) {
                // everything that does not depend on the operands first; the stage counter's load travels
                // while the dY barrier is polled
                const int ds = step & (kDyStages - 1);
                // B: atom 0 = the raw dY slab, atom 1 (N = 64 only) = its lo part, one slab further
                // (feature-major dY: K-major tile, 8-feature atoms 1 KiB apart; the lo tile continues the raw one)
                const uint64_t b_desc = kDyFm ? smem_desc_sw128(smem_base + kOffDy + ds * kDyStageBytes, 16, 1024)
                                              : smem_desc_mnmajor_sw128(smem_base + kOffDy + ds * kDyStageBytes, kSlabBytes);
                const uint32_t a_tm = tmem + kAccCols + as * kAStageCols;
                const uint32_t a_bar = a_empty(as), dy_bar = dy_empty(ds);
                const uint32_t a_cnt = a_count(as);
                const uint32_t seen = smem_load_acquire(a_cnt);
                wait(kPasses != 1 && !kIo16 ? dylo_full(ds) : dy_full(ds), (uint32_t)(step / kDyStages) & 1u);
                if ((int32_t)(seen - a_target) < 0) wait_count(a_cnt, a_target);
                // the split warps' tcgen05.st (and the drain warps' tcgen05.ld of the columns) precede the MMAs
                tc_fence_after();
                if (elect_one() & (bad == 0)) {
                    if (kPasses == 5) {
                        // [hi tile ; lo tile]: two atoms of 32 features along N, 2 KiB apart; 16 tokens = 1 KiB per instruction
                        const uint64_t b16 = smem_desc_sw64(smem_base + kOffDy + ds * kDyStageBytes + kSlabBytes, kSlabBytes / 2, 512);
#pragma unroll
                        for (int s = 0; s < 2; ++s) {  // x_hi pairs in columns 0-15 of the stage, x_lo pairs in 16-31
                            const uint64_t b = b16 + (uint64_t)(s * (1024 >> 4));
                            mma_ts_f16(d, a_tm + s * 8, b, idesc_bf16_wide, s == 0 ? acc0 : 1u);   // x_hi x [dy_hi ; dy_lo]
                            mma_ts_f16(d + 32, a_tm + 16 + s * 8, b, idesc_bf16, 1u);              // x_lo x dy_hi
                        }
                    } else if (kBf16) {
                        // K-major bf16 tile made by the dY split warps, or (bf16 tensors) the box as TMA wrote it:
                        // atoms of 8 token rows x 64 bytes, 512 bytes apart along K, 16 tokens = 1 KiB per instruction
                        const uint64_t b16 =
                            kIo16 ? smem_desc_sw64(smem_base + kOffDy + ds * kDyStageBytes, kSlabBytes, 512)
                                  : smem_desc_noswizzle(smem_base + kOffDy + ds * kDyStageBytes + kSlabBytes, kImage16Lbo, kImage16Sbo);
#pragma unroll
                        for (int s = 0; s < 2; ++s)  // 16 tokens per instruction: 8 columns of token pairs
                            mma_ts_f16(d, a_tm + s * 8, b16 + (uint64_t)(s * (kImage16StepBytes >> 4)), idesc_bf16,
                                       s == 0 ? acc0 : 1u);
                    } else {
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            // k-step s = 8 tokens: 8 rows of 128 bytes further (token-major) or 32 bytes further inside
                            // the swizzled rows (feature-major)
                            const uint64_t b = b_desc + (uint64_t)(kDyFm ? s * 2 : s * (kKStepBytes >> 4));
                            if (kPasses == 3) {
                                mma_ts_tf32(d, a_tm + s * 8, b, idesc_wide, s == 0 ? acc0 : 1u);     // x x [dy ; dy_lo]
                                mma_ts_tf32(d + 32, a_tm + 32 + s * 8, b, idesc_narrow, 1u);         // x_lo x dy
                            } else {
                                mma_ts_tf32(d, a_tm + s * 8, b, idesc_narrow, s == 0 ? acc0 : 1u);
                            }
                        }
                    }
                    mma_commit(a_bar);
                    mma_commit(dy_bar);
                    // the segment's columns are complete once everything this thread issued has executed
                    if (step + 1 == seg_end) mma_commit(p_bar);
                }
                acc0 = 1u;
                const int next = as + nchunks;
                const bool wrap = next >= kStages;
                as = wrap ? next - kStages : next;
                a_target += wrap ? 4u : 0u;
            }
        }
    } else if (warp < kFirstDrainWarp) {
        // ------------------------------------------------------------------ X split
        // Thread (quarter j, lane c) owns feature c of the unit's block j = tensor-memory lane 32 j + c and
        // reads that feature of the slab's 32 tokens: with the 128-byte swizzle (16-byte chunk index XOR
        // token mod 8) the 32 lanes of a warp hit 32 different banks.
        const int quarter = warp & 3;
        const int group = (warp - kFirstSplitWarp) >> 2;
        const uint32_t tmem_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        int xs = group;        // stage of unit u: u mod kStages, kept incrementally (u grows by kSplitGroups)
        uint32_t use = 0;      // u / kStages
        for (int u = group; u < nunits; u += kSplitGroups) {
            // one wait instruction for both barriers (a successful wait costs ~85 cycles whatever it tests): the
            // lower half-warp polls the slabs' arrival, the upper half the tensor-memory stage's release
            {
                const bool upper = lane >= 16;
                wait(upper ? a_empty(xs) : x_full(xs), (use & 1u) ^ (upper ? 1u : 0u));
                __syncwarp();
            }
            // (a quarter without a block, in an item's ragged last chunk, reads whatever the stage holds: its
            // accumulator rows are independent of the others and never stored)
            uint32_t hi[32], lo[32];
            {
                if (kIo16) {
                    // bf16 slab [token][feature], 64-byte rows, 64-byte swizzle (16-byte chunk index XOR (token / 2) mod 4)
                    const uint8_t* col = smem_gen + kOffX + xs * kXStageBytes + quarter * kSlabBytes + ((lane & 7) << 1);
#pragma unroll
                    for (int t = 0; t < 32; ++t)
                        hi[t] = *reinterpret_cast<const uint16_t*>(col + t * 64 + (((lane >> 3) ^ ((t >> 1) & 3)) << 4));
                } else if (kXFm) {
                    // the slab is [feature][token]: this thread's feature is row `lane`, 8 chunks of 4 tokens
                    const uint8_t* rowp = smem_gen + kOffX + xs * kXStageBytes + quarter * kSlabBytes + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 v4 = *reinterpret_cast<const uint4*>(rowp + ((j ^ (lane & 7)) << 4));
                        hi[4 * j + 0] = v4.x; hi[4 * j + 1] = v4.y; hi[4 * j + 2] = v4.z; hi[4 * j + 3] = v4.w;
                    }
#pragma unroll
                    for (int t = 0; t < 32; ++t)
                        if (kPasses == 3) lo[t] = __float_as_uint(__uint_as_float(hi[t]) - __uint_as_float(hi[t] & 0xffffe000u));
                } else {
                    const uint8_t* col = smem_gen + kOffX + xs * kXStageBytes + quarter * kSlabBytes + ((lane & 3) << 2);
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const uint32_t v = *reinterpret_cast<const uint32_t*>(col + t * 128 + (((lane >> 2) ^ (t & 7)) << 4));
                        hi[t] = v;
                        if (kPasses == 3) lo[t] = __float_as_uint(__uint_as_float(v) - __uint_as_float(v & 0xffffe000u));
                    }
                }
            }
            tc_fence_after();
            const uint32_t a_tm = tmem_lane + kAccCols + xs * kAStageCols;
            if (kPasses == 5) {
                uint32_t packed[32];  // columns 0-15: token pairs of hi = bf16(x); columns 16-31: of lo = bf16(x - hi)
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    split_bf16x2(__uint_as_float(hi[2 * j]), __uint_as_float(hi[2 * j + 1]), packed[j], packed[16 + j]);
                }
                tmem_st32(a_tm, packed);
            } else if (kBf16) {
                uint32_t packed[16];  // column j: token 2j in the low half, token 2j + 1 in the high half
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (kIo16) {
                        packed[j] = hi[2 * j] | (hi[2 * j + 1] << 16);
                    } else {
                        const __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(hi[2 * j]), __uint_as_float(hi[2 * j + 1]));
                        packed[j] = *reinterpret_cast<const uint32_t*>(&pr);
                    }
                }
                tmem_st16(a_tm, packed);
            } else {
                tmem_st32(a_tm, hi);
                if (kPasses == 3) tmem_st32(a_tm + 32, lo);
            }
            // The slabs are released only here: the stores above took every loaded value as an operand, so the loads
            // have returned.  Released right after the loads were issued, a refill (TMA, async proxy) has been seen
            // to overtake reads still queued in the load/store unit (generic proxy): a few rows of a slab were then
            // read from the next unit.  (The alternative, a proxy fence before the arrival, costs 3 % more.)
            mbar_arrive(x_empty(xs));
            tmem_wait_st();
            tc_fence_before();
            if ((lane == 0) & (bad == 0)) smem_add_release(a_count(xs), 1u);  // nothing is published once a wait has given up
            const bool wrap = xs + kSplitGroups >= kStages;
            xs = wrap ? xs + kSplitGroups - kStages : xs + kSplitGroups;
            use += wrap ? 1u : 0u;
        }
    } else {
        // ------------------------------------------------------------------ drain + epilogue
        const int quarter = warp & 3;  // block position inside the chunk = tensor-memory lane quarter
        const uint32_t tmem_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        // this thread's row (feature c = lane of block `quarter`) of chunk ch's master tile
        float* master = reinterpret_cast<float*>(smem_gen + kOffMaster) + (quarter * 32 + lane) * 32;
        const int swz = lane & 7;  // rotate 16-B chunks by the row so that a warp's accesses spread over banks
        for (int ch = 0; ch < nchunks; ++ch)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(master + ch * (kMasterBytes / 4) + ((j ^ swz) << 2)) =
                    make_float4(0.f, 0.f, 0.f, 0.f);

        uint32_t ready_ph = 0;
        bool ok = true;
        for (int step = 0; step < nsteps && ok; ++step) {
            if (!drain_step(step)) continue;
            for (int ch = 0; ch < nchunks; ++ch) {
                wait(p_ready(ch), (ready_ph >> ch) & 1u);
                ok = !__any_sync(0xffffffffu, bad != 0);
                if (!ok) break;
                ready_ph ^= 1u << ch;
                tc_fence_after();
                uint32_t acc[32], corr[32];
                tmem_ld32(tmem_lane + ch * kChunkCols, acc);
                if (kSplit) tmem_ld32(tmem_lane + ch * kChunkCols + 32, corr);
                tmem_wait_ld();
                if (!kSplit) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) corr[j] = 0u;
                }
                tc_fence_before();
                mbar_arrive(p_taken(ch));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4* mp = reinterpret_cast<float4*>(master + ch * (kMasterBytes / 4) + ((j ^ swz) << 2));
                    float4 v = *mp;
                    v.x += __uint_as_float(acc[j * 4 + 0]) + __uint_as_float(corr[j * 4 + 0]);
                    v.y += __uint_as_float(acc[j * 4 + 1]) + __uint_as_float(corr[j * 4 + 1]);
                    v.z += __uint_as_float(acc[j * 4 + 2]) + __uint_as_float(corr[j * 4 + 2]);
                    v.w += __uint_as_float(acc[j * 4 + 3]) + __uint_as_float(corr[j * 4 + 3]);
                    *mp = v;
                }
            }
        }

        if (ok && *abort_flag == 0) {
            float* out = p.out + (int64_t)blockIdx.y * p.split_stride;
            for (int ch = 0; ch < nchunks; ++ch) {
                const int nb = min(4, nblk - ch * 4);
                const int slot = __shfl_sync(0xffffffffu, my_ent.y, ch * 4 + min(quarter, 3));
                if (quarter >= nb) continue;  // warp-uniform
                float4* dst = reinterpret_cast<float4*>(out + ((int64_t)slot * 32 + lane) * 32);
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 v = *reinterpret_cast<const float4*>(master + ch * (kMasterBytes / 4) + ((j ^ swz) << 2));
                    dst[j] = v;
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                if (p.block_sumsq != nullptr) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0) p.block_sumsq[slot] = ss;
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicOr(p.status, 1u);
    if (warp == kFirstMmaWarp) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// item table from the CSR offsets: every row is cut into segments of at most kItemBlocks blocks
__global__ void __launch_bounds__(256)
sddmm_items_kernel(const int32_t* __restrict__ ptr, int n_rows, int32_t* __restrict__ items) {
    __shared__ int running;
    __shared__ int scan[256];
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < n_rows; base += 256) {
        const int r = base + threadIdx.x;
        const int cnt = r < n_rows ? ptr[r + 1] - ptr[r] : 0;
        const int mine = (cnt + kItemBlocks - 1) / kItemBlocks;
        scan[threadIdx.x] = mine;
        __syncthreads();
        for (int o = 1; o < 256; o <<= 1) {  // inclusive Hillis-Steele scan
            const int v = threadIdx.x >= o ? scan[threadIdx.x - o] : 0;
            __syncthreads();
            scan[threadIdx.x] += v;
            __syncthreads();
        }
        const int first = running + scan[threadIdx.x] - mine;
        for (int i = 0; i < mine; ++i) {
            int4 it;
            it.x = r;
            it.y = ptr[r] + i * kItemBlocks;
            it.z = min(kItemBlocks, cnt - i * kItemBlocks);
            it.w = 0;
            reinterpret_cast<int4*>(items + 4)[first + i] = it;
        }
        __syncthreads();
        if (threadIdx.x == 255) running += scan[255];
        __syncthreads();
    }
    if (threadIdx.x == 0) items[0] = running;
}

// out[i] = sum over splits of ws[s][i], in split order; optional per-slot sum of squares
__global__ void __launch_bounds__(256)
sddmm_reduce_kernel(const float* __restrict__ ws, int splits, int64_t split_stride, float* __restrict__ out,
                    float* __restrict__ block_sumsq) {
    __shared__ float red[8];
    const int64_t slot = blockIdx.x;
    const float* src = ws + slot * kBlockElems + threadIdx.x * 4;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + s * split_stride);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(out + slot * kBlockElems)[threadIdx.x] = acc;
    if (block_sumsq != nullptr) {
        float ss = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += red[w];
            block_sumsq[slot] = t;
        }
    }
}

// Scratch of bsmm_sddmm_static: the per-token-range partial results live here instead of in a
// caller-provided workspace.  Every GPU that loads the library holds these bytes until exit.
constexpr size_t kStaticScratchBytes = BSMM_SDDMM_STATIC_MAX_BYTES;
static __device__ __align__(256) unsigned char g_sddmm_static_scratch[kStaticScratchBytes];

int64_t max_items(int64_t n_rows, int64_t nnz) { return nnz / kItemBlocks + n_rows; }

// Token ranges.  Two constraints: enough CTAs for a few waves over 148 SMs, and a range whose slice of
// X and dY (tokens x (rows + cols) x 4 bytes) stays L2-resident (at most 64 MiB) while the successive
// waves of items walk it -- otherwise every wave streams the slice from HBM again.
void choose_splits(int64_t n_rows, int64_t cols, int64_t nnz, int64_t tokens, int64_t* splits,
                   int64_t* tokens_per_split) {
    int64_t est_items = (nnz + kItemBlocks - 1) / kItemBlocks;
    if (est_items < n_rows && nnz >= n_rows) est_items = n_rows;
    if (est_items < 1) est_items = 1;
    int64_t want = (4 * 148 + est_items - 1) / est_items;
    if (est_items > 148) {  // more than one wave per range: keep the range in L2
        const int64_t bytes_per_token = (n_rows * 32 + cols) * 4;
        const int64_t l2_tokens = (64ll << 20) / (bytes_per_token > 0 ? bytes_per_token : 1);
        const int64_t for_l2 = (tokens + l2_tokens - 1) / (l2_tokens > 0 ? l2_tokens : 1);
        if (for_l2 > want) want = for_l2 < 8 ? for_l2 : 8;  // bounded: every range costs a partial result
    }
    const int64_t max_splits = (tokens + 1023) / 1024;  // about 1024 tokens per range at least
    if (want > max_splits) want = max_splits;
    if (want < 1) want = 1;
    int64_t per = (tokens + want - 1) / want;
    per = (per + 255) / 256 * 256;
    *tokens_per_split = per;
    *splits = (tokens + per - 1) / per;
    if (*splits < 1) *splits = 1;
}

}  // namespace

// Device address of the static scratch array on the current device.  In host code the array's name
// is only a host-side stand-in for the symbol; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
cudaError_t sddmm_static_scratch(void** ptr, size_t* bytes) {
    constexpr int kMaxDevices = 64;
    static void* cache[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_sddmm_static_scratch);
        if (err != cudaSuccess) return err;
        cache[dev] = p;
    }
    *ptr = cache[dev];
    *bytes = kStaticScratchBytes;
    return cudaSuccess;
}

int64_t sddmm_plan_bytes(int64_t n_rows, int64_t nnz) { return 16 + 16 * max_items(n_rows, nnz); }

cudaError_t launch_build_sddmm_plan(const int32_t* ptr, int64_t n_rows, int64_t nnz, void* plan, cudaStream_t stream) {
    (void)nnz;
    sddmm_items_kernel<<<1, 256, 0, stream>>>(ptr, (int)n_rows, static_cast<int32_t*>(plan));
    return cudaGetLastError();
}

int64_t sddmm_umma_workspace_bytes(int64_t rows, int64_t cols, int64_t tokens, int64_t nnz, uint32_t precision) {
    if (!is_umma_precision(precision) || tokens < kStepTokens || nnz == 0) return 0;
    int64_t splits, per;
    choose_splits(rows / 32, cols, nnz, tokens, &splits, &per);
    return splits > 1 ? splits * nnz * (int64_t)kBlockElems * 4 : 0;
}

namespace {

template <int kPasses, bool kXFm, bool kDyFm>
cudaError_t launch_variant(dim3 grid, const CUtensorMap& tmap_x, const CUtensorMap& tmap_dy, const SddmmParams& p,
                           cudaStream_t stream) {
    // the shared-memory attribute is per device and kernel variant: set once each, then remembered
    constexpr int kMaxDevices = 64;
    static bool attribute_set[kMaxDevices] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!attribute_set[dev]) {
        err = cudaFuncSetAttribute(sddmm_umma_tf32_kernel<kPasses, kXFm, kDyFm>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (err != cudaSuccess) return err;
        attribute_set[dev] = true;
    }
    sddmm_umma_tf32_kernel<kPasses, kXFm, kDyFm><<<grid, kThreads, kSmemBytes, stream>>>(tmap_x, tmap_dy, p);
    return cudaGetLastError();
}

template <int kPasses>
cudaError_t launch_layout(bool x_fm, bool dy_fm, dim3 grid, const CUtensorMap& tmap_x, const CUtensorMap& tmap_dy,
                          const SddmmParams& p, cudaStream_t stream) {
    if (x_fm) return dy_fm ? launch_variant<kPasses, true, true>(grid, tmap_x, tmap_dy, p, stream)
                           : launch_variant<kPasses, true, false>(grid, tmap_x, tmap_dy, p, stream);
    return dy_fm ? launch_variant<kPasses, false, true>(grid, tmap_x, tmap_dy, p, stream)
                 : launch_variant<kPasses, false, false>(grid, tmap_x, tmap_dy, p, stream);
}

}  // namespace

// a = dY, b = X; *_feature_major: the tensor is [features, tokens] contiguous instead of [tokens, features];
// io_bf16: both are bf16 tensors (token-major, BSMM_PREC_BF16)
cudaError_t launch_sddmm_umma(const void* a, bool a_feature_major, const void* b, bool b_feature_major, int64_t rows,
                              int64_t cols, int64_t tokens, float* sparse_c, const int32_t* csr_idx, const void* plan,
                              int64_t nnz, float* block_sumsq, void* workspace, uint32_t precision, bool io_bf16,
                              cudaStream_t stream) {
    if (io_bf16 && (precision != BSMM_PREC_BF16 || a_feature_major || b_feature_major)) return cudaErrorNotSupported;
    if (!is_umma_precision(precision) || plan == nullptr || csr_idx == nullptr) return cudaErrorNotSupported;
    if (tokens < kStepTokens) return cudaErrorNotSupported;  // a box may not exceed its tensor
    // a feature-major tensor has rows of `tokens` floats: the tensor map wants that pitch to be a multiple of 16 bytes
    if ((a_feature_major || b_feature_major) && (tokens % 4) != 0) return cudaErrorNotSupported;
    if (tokens > 0x7fffffffll) return cudaErrorInvalidValue;
    const int64_t n_rows = rows / 32;
    int64_t splits, per;
    choose_splits(n_rows, cols, nnz, tokens, &splits, &per);
    if (splits > 1 && workspace == nullptr) return cudaErrorInvalidValue;
    if (splits > 65535) return cudaErrorInvalidValue;

    // the bf16 hi | lo kernel takes token-major operands; feature-major ones compute as 3xTF32 (same accuracy class)
    const bool x5 = precision == BSMM_PREC_BF16X3 && !a_feature_major && !b_feature_major;
    const bool x3 = precision == BSMM_PREC_TF32X3 || (precision == BSMM_PREC_BF16X3 && !x5);
    const bool bf16 = precision == BSMM_PREC_BF16;
    CUtensorMap tmap_x, tmap_dy;
    cudaError_t err;
    if (io_bf16) {
        err = make_tmap_2d(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b, (uint64_t)cols, (uint64_t)tokens, 32, kStepTokens,
                           CU_TENSOR_MAP_SWIZZLE_64B);
        if (err != cudaSuccess) return err;
        err = make_tmap_2d(&tmap_dy, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, (uint64_t)rows, (uint64_t)tokens, 32, kStepTokens,
                           CU_TENSOR_MAP_SWIZZLE_64B);
    } else if (b_feature_major)
        err = make_tmap_2d(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, b, (uint64_t)tokens, (uint64_t)cols, kStepTokens, 32,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    else
        err = make_tmap_2d(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, b, (uint64_t)cols, (uint64_t)tokens, 32,
                           kStepTokens, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess) return err;
    // token-major dY is the MMA's operand as loaded in the tf32 modes (32-byte-atom swizzle); in bf16 mode a warp
    // reads it.  Feature-major dY is the K-major canonical tile under the plain 128-byte swizzle in every mode.
    if (io_bf16)
        ;  // both maps were made above
    else if (a_feature_major)
        err = make_tmap_2d(&tmap_dy, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a, (uint64_t)tokens, (uint64_t)rows, kStepTokens, 32,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    else
        err = make_tmap_2d(&tmap_dy, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a, (uint64_t)rows, (uint64_t)tokens, 32,
                           kStepTokens, (bf16 || x5) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (err != cudaSuccess) return err;

    SddmmParams p;
    p.items = static_cast<const int32_t*>(plan);
    p.idx = reinterpret_cast<const int2*>(csr_idx);
    p.out = splits > 1 ? static_cast<float*>(workspace) : sparse_c;
    p.block_sumsq = splits > 1 ? nullptr : block_sumsq;
    err = device_status_address(&p.status);
    if (err != cudaSuccess) return err;
    p.tokens = tokens;
    p.tokens_per_split = per;
    p.split_stride = nnz * (int64_t)kBlockElems;
    dim3 grid((unsigned)max_items(n_rows, nnz), (unsigned)splits);
    if (x3) err = launch_layout<3>(b_feature_major, a_feature_major, grid, tmap_x, tmap_dy, p, stream);
    else if (x5) err = launch_variant<5, false, false>(grid, tmap_x, tmap_dy, p, stream);
    else if (io_bf16) err = launch_variant<4, false, false>(grid, tmap_x, tmap_dy, p, stream);
    else if (bf16) err = launch_layout<0>(b_feature_major, a_feature_major, grid, tmap_x, tmap_dy, p, stream);
    else err = launch_layout<1>(b_feature_major, a_feature_major, grid, tmap_x, tmap_dy, p, stream);
    if (err != cudaSuccess) return err;
    if (splits > 1) {
        sddmm_reduce_kernel<<<(unsigned)nnz, 256, 0, stream>>>(static_cast<const float*>(workspace), (int)splits,
                                                               p.split_stride, sparse_c, block_sumsq);
        err = cudaGetLastError();
    }
    return err;
}

}  // namespace bsmm
