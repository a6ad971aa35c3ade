// Tensor-core dense x block-sparse -> dense kernel for sm_100a (forward and dgrad of one
// block-sparse Linear; replaces the reference's cutlass::gemm::kernel<block_task>,
// cutlass/gemm/dispatch.h:185-218 and block_task.h:647-715).
//
// Tile: 128 tokens x G output block-rows (G*32 columns), accumulated in tensor memory.  The
// contraction axis is walked one 32-wide activation slab at a time, visiting only slabs for which
// the group has at least one block (the plan lists them, bsmm_plan.cu).  The kernel is persistent:
// one CTA per SM walks its tiles, and every ring position runs on across tiles.
//
//   warps 0-3   weight producers : warp w feeds MMA warp w's own ring of kWRing stages, one linear bulk
//                                  copy (8 KiB, bf16: 2 KiB) per block of its packed weight image, and beside it
//                                  a 32-byte command: everything the MMA warp needs to know about the block
//                                  (accumulator and operand addresses, barriers, flags), so that the plan is
//                                  decoded off the MMA warps' critical path
//   warp 4      activation producer : TMA tensor load of the [128 x 32] fp32 slab (128-byte swizzle)
//   warps 5-8   MMA : tcgen05.mma kind::tf32, M = 128, A from tensor memory, B from smem; output row r
//                     of the group belongs to warp r mod 4.
//                     3xTF32, per k-step (8 values of k) two instructions:
//                       x_hi x [w_hi ; w_lo]  (N = 64) -> main | correction columns of the row
//                       x_lo x  w_hi          (N = 32) -> correction columns
//                     single-pass TF32: one N = 32 instruction per k-step.
//                     bf16 hi | lo (BSMM_PREC_BF16X3): the same two instructions per k-step as 3xTF32, kind::f16
//                     on bf16 parts hi = bf16(v), lo = bf16(v - hi), with k-steps of 16: half as many instructions
//   warps 9-16  split : two groups of four, alternate slabs: slab smem -> registers -> tensor memory
//                       (lane = token, column = k) with tcgen05.st, which makes it the MMA's A operand;
//                       for 3xTF32 also lo = x - trunc_tf32(x) (the tensor core reads only the tf32
//                       bits of an operand, so the raw slab is x_hi)
//   warps 17-20 drain : after every kDrainEvery-th block of a row and after its last one,
//                       tcgen05.ld the row's columns, main + correction (+ bias) into a staging tile in
//                       shared memory, which one thread sends off with a TMA store (the row's first
//                       promotion in the tile) or a TMA add-reduction (later ones)
//
// Measured on an idle SM, one block costs the tensor pipe 255 clk (3xTF32) or 165 clk (single pass)
// in this form, against 422 / 232 clk with A read from shared memory (4 KiB per instruction).
// Keeping the main term apart from the corrections and promoting it every 48 blocks bounds the
// tensor core's systematic fp32-accumulate error (about 2e-8 relative per accumulation).
// Every wait is bounded; on expiry the CTA raises the device status word, stops issuing and drains.
#include <cuda_bf16.h>

#include "bsmm_ptx.cuh"
#include "bsmm_umma.cuh"

namespace bsmm {

__device__ unsigned int g_device_status = 0;

namespace {

using namespace ptx;

constexpr int kTileTokens = 128;
constexpr uint32_t kSlabBytes = kTileTokens * 32 * 4;  // 16 KiB: [128 tokens][32 k] fp32
constexpr uint32_t kWStageBytes = kImage32Bytes;       // 8 KiB: hi and lo parts interleaved
constexpr uint32_t kTmemCols = 512;
constexpr int kMmaWarps = kDsdMmaWarps;
static_assert(kMmaWarps == 4, "a row's number is its warp's number plus 0 or 4");
constexpr int kWProducers = kMmaWarps;            // warp w loads the weight blocks of MMA warp w
constexpr int kXProducerWarp = kWProducers;       // this warp loads activation slabs
constexpr int kFirstMmaWarp = kXProducerWarp + 1;
constexpr int kFirstSplitWarp = kFirstMmaWarp + kMmaWarps;
// then the split warps (Cfg::kSplitGroups groups of four) and four drain warps

template <int G, int kPasses>
struct Cfg {
    // kPasses: 3 = 3xTF32, 1 = single-pass TF32, 0 = bf16 operands (kind::f16) rounded in the kernel from fp32
    // tensors, 4 = bf16 operands with bf16 activations and outputs in memory, 5 = three products of bf16 hi and lo
    // parts of fp32 tensors (the 3xTF32 scheme with kind::f16 instructions: two k-steps of 16 instead of four of 8);
    // fp32 accumulation throughout
    static constexpr bool kBf16 = kPasses == 0 || kPasses == 4 || kPasses == 5;
    static constexpr bool kIo16 = kPasses == 4;
    static constexpr bool kSplit = kPasses == 3 || kPasses == 5;       // hi and lo parts, correction columns
    static constexpr uint32_t kRowCols = kSplit ? 64 : 32;     // main | correction
    static constexpr uint32_t kAStageCols = kPasses == 3 ? 64 : (kPasses == 1 || kPasses == 5) ? 32 : 16;  // x_hi | x_lo; bf16 pairs
    static constexpr uint32_t kWBytes = kPasses == 5 ? kImage16x3Bytes : kBf16 ? kImage16Bytes : kImage32Bytes;    // one block's image
    static constexpr uint32_t kAccCols = G * kRowCols;
    static constexpr int kAStagesMax = (int)((kTmemCols - kAccCols) / kAStageCols);
    static constexpr int kAStages = kAStagesMax >= 8 ? 8 : kAStagesMax >= 4 ? 4 : kAStagesMax;  // 8, 4, 3 or 2
    // Split-warp groups take slabs round-robin; a ring stage must always meet the same group, so the stage
    // counts are multiples of the group count.  Three stages get three groups: one stage each.
    static constexpr int kSplitGroups = kAStages % 3 == 0 ? 3 : 2;
    static constexpr int kXStages = 2 * kSplitGroups;
    static constexpr int kFirstDrainWarp = kFirstSplitWarp + 4 * kSplitGroups;
    static constexpr int kThreads = 32 * (kFirstDrainWarp + 4);
    static_assert(kAStages % kSplitGroups == 0, "a ring stage must stay with one split-warp group");
    // Weight stages per MMA warp (a ring of its own, a power of two).  Single-pass TF32 spends the least tensor
    // time per 8 KiB image and gains 11 % from four stages where shared memory has room for them, the bf16 hi | lo
    // mode 2 %; 3xTF32 (-1 %) and bf16 (0 %) keep two.
    static constexpr int kWRing =
        ((kPasses == 1 || kPasses == 5) && (kXStages + 2) * kSlabBytes + 4 * kMmaWarps * kWStageBytes + 2048 <= 232448) ? 4 : 2;
    static constexpr int kWStages = kMmaWarps * kWRing;
    static constexpr uint32_t kOffX = 0;
    static constexpr uint32_t kOffW = kOffX + kXStages * kSlabBytes;
    static constexpr uint32_t kOffOut = kOffW + kWStages * kWStageBytes;   // two staging tiles of the epilogue
    static constexpr uint32_t kOffBar = kOffOut + 2 * kSlabBytes;
    static constexpr int kNumBars = 2 * kXStages + 2 * kWStages + kAStages + 2 * G;
    static constexpr uint32_t kOffMisc = kOffBar + kNumBars * 8;
    static constexpr uint32_t kOffCmd = (kOffMisc + 64 + 15) / 16 * 16;   // one 32-byte command per weight stage
    static constexpr uint32_t kSmemBytes = kOffCmd + kWStages * 32 + 1024;  // + slack to align the base to 1 KiB
    static_assert(kAStages >= 2, "tensor memory over-subscribed");
    static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");
};

// Further output tensors (peer GPUs' buffers reached through NVLink; plain TMA stores).  Broadcast mode: the same
// tiles are stored to each of them.  Scatter mode: map[i] is rank i's tensor of parts, and a completed tile is
// stored into this rank's slot of the tensor of the rank that owns the tile's rows.
constexpr int kMaxPeerOutputs = 8;
struct PeerMaps {
    CUtensorMap map[kMaxPeerOutputs];
};

struct DsdParams {
    const uint8_t* packed;      // weight images of this orientation, slot-major
    const int32_t* group_off;   // [groups + 1]
    const int32_t* group_slabs; // [groups]
    const PlanEntry* entries;
    const float* bias;          // may be null
    const float* residual;      // may be null: [m, n] row-major, added with the bias (row-major output only)
    float* pre_act;             // may be null: [m, n] row-major, receives the sum before the activation
    int32_t act;                // 0 none, 1 GELU: applied to a row's completed sum (row-major output only)
    int32_t n_peers;            // further output tensors (other GPUs' copies of the output) that receive every completed tile
    int64_t out_ld;             // row pitch of the output tensor(s) in elements (n, or the full width when this call
    int64_t out_col0;           //   writes a column slice starting at out_col0)
    int64_t scatter_rows;       // > 0: scatter mode, rows per owner
    int32_t scatter_slot;       //      this rank's slot in the owners' tensors of parts
    float* out;                 // (bf16 in the bf16-tensor variant, which writes only through tmap_out)
    unsigned int* status;       // device status word
    int64_t m, n;
    int32_t n_out_blocks, groups;
    int32_t n_tiles;            // groups x token tiles; CTA b works on tiles b, b + gridDim.x, ...
    int32_t out_colmajor;
    uint32_t x_bytes;           // bytes one activation-slab load delivers: min(128, m) rows of 128 B
    long long* trace;           // diagnostics: 32 wait-cycle counters of CTA `trace_block`, or null
    int32_t trace_block;
};

// Counters written when tracing: cycles the role spent inside each kind of wait, and its loop total.
enum TraceSlot {
    kTrProdXEmpty = 0, kTrProdWEmpty, kTrProdTotal, kTrProdIssue,
    kTrMmaAFull = 4, kTrMmaWFull, kTrMmaPTaken, kTrMmaTotal,
    kTrMmaIssue = 14,
    kTrXfXFull = 8, kTrXfAEmpty, kTrXfTotal,
    kTrDrainPReady = 12, kTrDrainTotal,
};

// Out of line: the erf expansion would otherwise be inlined 32 times into the epilogue and cost the whole
// kernel registers that its hot loops want.
__device__ __noinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

template <int G, int kPasses>
__global__ void __launch_bounds__((Cfg<G, kPasses>::kThreads), 1)
dsd_umma_tf32_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_out,
                     const __grid_constant__ CUtensorMap tmap_pre, const __grid_constant__ PeerMaps peers,
                     const DsdParams p) {
    using C = Cfg<G, kPasses>;
    constexpr bool kBf16 = C::kBf16, kIo16 = C::kIo16, kSplit = C::kSplit;
    // bf16 tensors need no promotion against accumulation drift: a row is drained once, at its end
    constexpr int32_t kDrainFlag = kIo16 ? kPlanRowEnd : kPlanDrain;
    constexpr int XS = C::kXStages;
    constexpr int kFirstDrainWarp = C::kFirstDrainWarp;
    constexpr int kSplitGroups = C::kSplitGroups;
    constexpr int AS = C::kAStages;
    constexpr int kWRing = C::kWRing, kWStages = C::kWStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t bar0 = smem_base + C::kOffBar;
    auto x_full = [&](int s) { return bar0 + 8u * s; };                      // TMA delivered the slab
    auto x_empty = [&](int s) { return bar0 + 8u * (XS + s); };              // transform warps read it
    auto w_full = [&](int s) { return bar0 + 8u * (2 * XS + s); };
    auto w_empty = [&](int s) { return bar0 + 8u * (2 * XS + kWStages + s); };
    auto a_empty = [&](int s) { return bar0 + 8u * (2 * XS + 2 * kWStages + s); };  // every MMA warp is past the slab
    auto p_ready = [&](int r) { return bar0 + 8u * (2 * XS + 2 * kWStages + AS + r); };
    auto p_taken = [&](int r) { return bar0 + 8u * (2 * XS + 2 * kWStages + AS + G + r); };
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kOffMisc);
    // misc[0]: tensor-memory base address, misc[1]: abort flag, misc[2 + stage]: how many split warps have
    // completed a copy into that tensor-memory stage so far -- its u-th slab may be read at 4 * (u + 1)
    auto a_count = [&](int s) { return smem_base + C::kOffMisc + 8u + 4u * s; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < XS; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 128); }
        for (int s = 0; s < AS; ++s) mbar_init(a_empty(s), kMmaWarps);
        for (int s = 0; s < kWStages; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1); }
        for (int r = 0; r < G; ++r) { mbar_init(p_ready(r), 1); mbar_init(p_taken(r), 128); }
        misc[1] = 0;
        for (int s = 0; s < AS; ++s) misc[2 + s] = 0;
        fence_mbar_init();
    }
    if (warp == kFirstMmaWarp) {
        tmem_alloc(smem_base + C::kOffMisc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    volatile uint32_t* abort_flag = &misc[1];

#ifdef BSMM_TRACE
    const bool tracing = p.trace != nullptr && (int)blockIdx.x == p.trace_block;
#else
    constexpr bool tracing = false;
#endif
    long long tr[4] = {0, 0, 0, 0};
    const long long t_role0 = tracing ? clock64() : 0;
    // Waits never branch on their result in the common case: a conditional branch costs a lone warp ~40 cycles.
    // A wait that gives up (bounded, see mbar_wait) sets `bad`; the issuing instructions are predicated on it
    // and the role loops test it once per chunk, slab or promotion.
    uint32_t bad = 0;
    auto wait = [&](uint32_t bar, uint32_t parity, int which) {
        const long long t = tracing ? clock64() : 0;
        if (!mbar_try_wait(bar, parity) && !mbar_wait(bar, parity, abort_flag)) bad = 1;
        if (tracing) tr[which] += clock64() - t;
    };
    // bounded like mbar_wait: polls until the counter at `addr` has reached `target`
    auto wait_count = [&](uint32_t addr, uint32_t target) {
        const long long t = tracing ? clock64() : 0;
        if ((int32_t)(smem_load_acquire(addr) - target) < 0) {
            const long long t0 = clock64();
            for (;;) {
                if ((int32_t)(smem_load_acquire(addr) - target) >= 0) break;
                if (*abort_flag != 0) { bad = 1; break; }
                if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; bad = 1; break; }
            }
        }
        if (tracing) tr[0] += clock64() - t;
    };
    // The kernel is persistent: CTA b works on tiles b, b + gridDim.x, ...  (tile = group of G output
    // block-rows x 128 tokens), so the barrier and tensor-memory set-up is paid once and one tile's epilogue
    // overlaps the next tile's loads.  Every role walks the same tile sequence; ring positions (entry, slab
    // and promotion counts) run on across tiles.
    const int4* ents = reinterpret_cast<const int4*>(p.entries);
    const int n_tiles = p.n_tiles, tile_step = (int)gridDim.x;
    auto fetch = [&](int i, int end) { return i < end ? __ldg(ents + i) : make_int4(0, 0, 0, 0); };  // x inner, y slot, z row, w flags
    // The plan is read 32 entries per load (lane i holds entry base + i), one chunk ahead of use -- across
    // tile boundaries too: `ahead` is the chunk after (tile, base).
    auto prefetch = [&](int tile, int base, int e1) {
        if (base + 32 < e1) return fetch(base + 32 + lane, e1);
        const int nt = tile + tile_step;
        if (nt >= n_tiles) return make_int4(0, 0, 0, 0);
        const int ng = nt % p.groups;
        return fetch(__ldg(p.group_off + ng) + lane, __ldg(p.group_off + ng + 1));
    };
    // A tile without entries (G consecutive empty block-rows) has no chunk to walk, so nothing inside its chunk
    // loop moves `ahead` on: the role does it by hand, or the next tile would be decoded from this tile's empty chunk.
    auto skip_empty_tile = [&](int tile) {
        const int nt = tile + tile_step;
        if (nt >= n_tiles) return make_int4(0, 0, 0, 0);
        const int ng = nt % p.groups;
        return fetch(__ldg(p.group_off + ng) + lane, __ldg(p.group_off + ng + 1));
    };
    auto first_chunk = [&]() {
        if ((int)blockIdx.x >= n_tiles) return make_int4(0, 0, 0, 0);
        const int g0 = (int)blockIdx.x % p.groups;
        return fetch(__ldg(p.group_off + g0) + lane, __ldg(p.group_off + g0 + 1));
    };

    // Control warps are latency machines: one warp executing dependent scalar code retires an instruction
    // every few cycles, a conditional branch costs ~40 cycles, a successful barrier wait ~85 and a global load
    // ~1000, while the tensor core needs only ~200 cycles for a block.  Hence: the flag bits and row numbers
    // of a chunk become warp-uniform bit masks (ballots) and the per-entry decisions are bit tests; ring
    // stages follow from entry and slab counts, so a warp visits only the entries it has work for.
    // Command flags (word 7 of a command; words 0-6: accumulator columns, activation stage, its counter's
    // address and target, its release barrier, the row's p_ready and p_taken barriers)
    constexpr uint32_t kCmdAcc = 1u, kCmdWarpLast = 2u, kCmdDrain = 4u, kCmdIdleShift = 3u /* 2 bits */,
                       kCmdNeedTaken = 32u, kCmdTakenParity = 64u, kCmdEnd = 128u;
    auto cmd_addr = [&](int ws) { return smem_base + C::kOffCmd + 32u * ws; };

    if (warp < kWProducers) {
        // ------------------------------------------------------------------ weight producers
        // Every MMA warp has a ring of kWRing stages of its own, filled by a producer warp of its own in the
        // order of that warp's blocks: one producer and one consumer per ring, each seeing every phase (which a
        // phase-parity barrier needs), and a full ring stalls nobody else's loads.
        // The producer also decodes the plan for its MMA warp: which accumulator columns and activation stage the
        // block uses, whether it starts a partial sum, ends a slab or triggers a promotion, and which barriers
        // that involves -- all of it a function of the plan's order alone -- and hands the result over as a
        // 32-byte command in the stage (written before the arrival that opens the stage's phase, so the phase's
        // observer sees it).  The MMA warp's loop is then: wait for the stage, read the command, wait for the
        // activation stage, issue.  Measured on c3_d0.25: -4...-6 % in the single-pass and bf16 modes, -1 % in 3xTF32.
        const uint32_t mw = (uint32_t)warp;
        uint32_t seq = 0;       // blocks of this warp's MMA warp loaded so far
        uint32_t started = 0;   // bit r: the row's columns hold a partial sum of the current segment
        uint32_t pending = 0;   // bit r: a promotion of the row was requested; its next block must see it taken
        uint32_t taken_ph = 0;  // bit r: parity of the next p_taken[r] phase to wait for
        int slab_base = -1;     // number (over all tiles of this CTA) of the last slab opened before this chunk
        int4 ahead = first_chunk();
        for (int tile = blockIdx.x; tile < n_tiles && !bad; tile += tile_step) {
            const int g = tile % p.groups;
            const int e0 = __ldg(p.group_off + g), e1 = __ldg(p.group_off + g + 1);
            if (e0 == e1) ahead = skip_empty_tile(tile);
            for (int base = e0; base < e1 && !bad; base += 32) {
                const int4 mine = ahead;
                ahead = prefetch(tile, base, e1);
                const uint32_t valid = __ballot_sync(0xffffffffu, base + lane < e1);
                const uint32_t firsts = __ballot_sync(0xffffffffu, (mine.w & kPlanFirst) != 0);
                const uint32_t lasts = __ballot_sync(0xffffffffu, (mine.w & kPlanLast) != 0);
                const uint32_t wlasts = __ballot_sync(0xffffffffu, (mine.w & kPlanWarpLast) != 0);
                const uint32_t drains = __ballot_sync(0xffffffffu, (mine.w & kDrainFlag) != 0);
                const uint32_t idle_b0 = __ballot_sync(0xffffffffu, (mine.w & (1 << kPlanIdleShift)) != 0);
                const uint32_t idle_b1 = __ballot_sync(0xffffffffu, (mine.w & (2 << kPlanIdleShift)) != 0);
                const uint32_t row_b2 = __ballot_sync(0xffffffffu, (mine.z & 4) != 0);
                uint32_t todo = __ballot_sync(0xffffffffu, ((uint32_t)mine.z & (kMmaWarps - 1)) == mw) & valid;
                while (todo != 0) {
                    const int i = __ffs(todo) - 1;
                    todo &= todo - 1;
                    const int slot = __shfl_sync(0xffffffffu, mine.y, i);
                    const int slab = slab_base + __popc(firsts & (0xffffffffu >> (31 - i)));
                    const int as = slab % AS;
                    const int ws = (int)(mw * kWRing + (seq & (kWRing - 1)));
                    const uint32_t row = mw | (((row_b2 >> i) & 1u) << 2);  // this warp's rows: mw and mw + 4
                    const uint32_t rbit = 1u << row;
                    const bool drain = ((drains >> i) & 1u) != 0;
                    // the warp that issues a slab's last block also arrives for the warps that have none in it
                    const uint32_t idle = ((lasts >> i) & 1u) * (((idle_b0 >> i) & 1u) | (((idle_b1 >> i) & 1u) << 1));
                    uint32_t flags = ((started & rbit) ? kCmdAcc : 0u) | (((wlasts >> i) & 1u) ? kCmdWarpLast : 0u) |
                                     (drain ? kCmdDrain : 0u) | (idle << kCmdIdleShift);
                    if (pending & rbit) {  // the drain warps must have read the row before it is overwritten
                        flags |= kCmdNeedTaken | (((taken_ph >> row) & 1u) ? kCmdTakenParity : 0u);
                        taken_ph ^= rbit;
                        pending &= ~rbit;
                    }
                    started |= rbit;
                    if (drain) { pending |= rbit; started &= ~rbit; }
                    const uint32_t c_d = tmem + row * C::kRowCols;
                    const uint32_t c_a = tmem + C::kAccCols + as * C::kAStageCols;
                    const uint32_t c_cnt = a_count(as), c_target = 4u * (uint32_t)(slab / AS + 1);
                    const uint32_t c_abar = a_empty(as), c_pbar = p_ready(row), c_taken = p_taken(row);
                    wait(w_empty(ws), ((seq / kWRing) & 1u) ^ 1u, 1);
                    ++seq;
                    const uint8_t* src = p.packed + (int64_t)slot * C::kWBytes;
                    if (elect_one() && !bad) {
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cmd_addr(ws)), "r"(c_d), "r"(c_a),
                                     "r"(c_cnt), "r"(c_target) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cmd_addr(ws) + 16u), "r"(c_abar),
                                     "r"(c_pbar), "r"(c_taken), "r"(flags) : "memory");
                        mbar_arrive_expect_tx(w_full(ws), C::kWBytes);
                        bulk_load(smem_base + C::kOffW + ws * kWStageBytes, src, C::kWBytes, w_full(ws));
                    }
                }
                slab_base += __popc(firsts & valid);
            }
        }
        {   // the end of this warp's blocks: a command without data
            const int ws = (int)(mw * kWRing + (seq & (kWRing - 1)));
            if (!bad) wait(w_empty(ws), ((seq / kWRing) & 1u) ^ 1u, 1);
            if (elect_one() && !bad) {
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %2};" ::"r"(cmd_addr(ws) + 16u), "r"(0u), "r"(kCmdEnd) : "memory");
                mbar_arrive(w_full(ws));
            }
        }
        if (tracing && lane == 0 && warp == 0) {
            p.trace[kTrProdWEmpty] = tr[1];
            p.trace[kTrProdTotal] = clock64() - t_role0;
        }
    } else if (warp == kXProducerWarp) {
        // ------------------------------------------------------------------ activation producer
        int xs = 0;
        uint32_t xph = 0;
        int4 ahead = first_chunk();
        for (int tile = blockIdx.x; tile < n_tiles && !bad; tile += tile_step) {
            const int g = tile % p.groups;
            const int32_t tok0 = (tile / p.groups) * kTileTokens;
            const int e0 = __ldg(p.group_off + g), e1 = __ldg(p.group_off + g + 1);
            if (e0 == e1) ahead = skip_empty_tile(tile);
            for (int base = e0; base < e1 && !bad; base += 32) {
                const int4 mine = ahead;
                ahead = prefetch(tile, base, e1);
                uint32_t firsts = __ballot_sync(0xffffffffu, (mine.w & kPlanFirst) != 0);
                while (firsts != 0) {
                    const int i = __ffs(firsts) - 1;
                    firsts &= firsts - 1;
                    wait(x_empty(xs), xph ^ 1u, 0);
                    const int inner = __shfl_sync(0xffffffffu, mine.x, i);
                    if (elect_one() && !bad) {
                        mbar_arrive_expect_tx(x_full(xs), p.x_bytes);
                        tma_load_2d(smem_base + C::kOffX + xs * kSlabBytes, &tmap_a, inner * 32, tok0, x_full(xs));
                    }
                    if (++xs == XS) { xs = 0; xph ^= 1u; }
                }
            }
        }
        if (tracing && lane == 0) p.trace[kTrProdXEmpty] = tr[0];
    } else if (warp < kFirstSplitWarp) {
        // ------------------------------------------------------------------ MMA issuers
        // The warps share the issue work by output row (row mod kMmaWarps): accumulations into one row stay
        // in one thread's program order, and while one warp is between blocks the others keep the tensor pipe
        // fed.  Each warp sees only its own blocks, as commands from its weight producer; a slab's stage is
        // released by one commit from every warp that read it plus, from the warp issuing the slab's last block,
        // plain arrivals on behalf of the warps that had nothing in it.
        const uint32_t mw = (uint32_t)(warp - kFirstMmaWarp);
        constexpr uint32_t idesc_wide = make_idesc(2u, 128u, 64u, false, false);
        constexpr uint32_t idesc_narrow = make_idesc(2u, 128u, 32u, false, false);
        constexpr uint32_t idesc_bf16 = make_idesc(1u, 128u, 32u, false, false);
        constexpr uint32_t idesc_bf16_wide = make_idesc(1u, 128u, 64u, false, false);
        static_assert((kWRing & (kWRing - 1)) == 0, "ring positions are taken with a mask");
        const uint32_t w0 = smem_base + C::kOffW + (mw * kWRing) * kWStageBytes;
        // descriptor of the ring's first stage; a stage further is kWStageBytes / 16 more in its address field
        const uint64_t b_desc0 = kPasses == 5 ? smem_desc_noswizzle(w0, kImage16x3Lbo, kImage16x3Sbo)
                                 : kBf16      ? smem_desc_noswizzle(w0, kImage16Lbo, kImage16Sbo)
                                              : smem_desc_noswizzle(w0, kImage32Lbo, kImage32Sbo);
        for (uint32_t seq = 0;; ++seq) {
            const uint32_t pos = seq & (uint32_t)(kWRing - 1);
            const int ws = (int)(mw * kWRing + pos);
            wait(w_full(ws), (seq / kWRing) & 1u, 1);
            uint32_t c_d, c_a, c_cnt, c_target, c_abar, c_pbar, c_taken, flags;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c_d), "=r"(c_a), "=r"(c_cnt), "=r"(c_target)
                         : "r"(cmd_addr(ws)) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c_abar), "=r"(c_pbar), "=r"(c_taken), "=r"(flags)
                         : "r"(cmd_addr(ws) + 16u) : "memory");
            if ((flags & kCmdEnd) | bad) break;
            const uint32_t seen = smem_load_acquire(c_cnt);
            if (flags & kCmdNeedTaken) wait(c_taken, (flags & kCmdTakenParity) ? 1u : 0u, 2);
            if ((int32_t)(seen - c_target) < 0) wait_count(c_cnt, c_target);
            // the split warps' tcgen05.st (and the drain warps' tcgen05.ld of the row) precede the MMAs
            tc_fence_after();
            const long long ti = tracing ? clock64() : 0;
            const uint64_t b_desc = b_desc0 + (uint64_t)(pos * (kWStageBytes >> 4));
            const uint32_t acc0 = flags & kCmdAcc;
            if (elect_one() & (bad == 0)) {
                if (kPasses == 5) {
#pragma unroll
                    for (int s = 0; s < 2; ++s) {  // k-step of 16: x_hi pairs in columns 0-15 of the stage, x_lo pairs in 16-31
                        const uint64_t b = b_desc + (uint64_t)(s * (kImage16x3StepBytes >> 4));
                        mma_ts_f16(c_d, c_a + s * 8, b, idesc_bf16_wide, s == 0 ? acc0 : 1u);   // x_hi x [w_hi ; w_lo]
                        mma_ts_f16(c_d + 32, c_a + 16 + s * 8, b, idesc_bf16, 1u);              // x_lo x w_hi
                    }
                } else if (kBf16) {
#pragma unroll
                    for (int s = 0; s < 2; ++s)  // k-step of 16: 8 columns (bf16 pairs) further, two k-chunks further
                        mma_ts_f16(c_d, c_a + s * 8, b_desc + (uint64_t)(s * (kImage16StepBytes >> 4)), idesc_bf16,
                                   s == 0 ? acc0 : 1u);
                } else {
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        // k-step s: 8 columns further in the slab's tensor-memory copy, 2 KiB further in the image
                        const uint64_t b = b_desc + (uint64_t)(s * (kImage32StepBytes >> 4));
                        const uint32_t acc = s == 0 ? acc0 : 1u;
                        if (kPasses == 3) {
                            mma_ts_tf32(c_d, c_a + s * 8, b, idesc_wide, acc);               // x_hi x [w_hi ; w_lo]
                            mma_ts_tf32(c_d + 32, c_a + 32 + s * 8, b, idesc_narrow, 1u);    // x_lo x w_hi
                        } else {
                            mma_ts_tf32(c_d, c_a + s * 8, b, idesc_narrow, acc);
                        }
                    }
                }
                mma_commit(w_empty(ws));
                if (flags & kCmdWarpLast) mma_commit(c_abar);
                const uint32_t idle = (flags >> kCmdIdleShift) & 3u;
                if (idle != 0) mbar_arrive_n(c_abar, idle);
                if (flags & kCmdDrain) mma_commit(c_pbar);
            }
            if (tracing) tr[3] += clock64() - ti;
        }
        if (tracing && lane == 0 && mw == 0) {
            p.trace[kTrMmaAFull] = tr[0];
            p.trace[kTrMmaWFull] = tr[1];
            p.trace[kTrMmaPTaken] = tr[2];
            p.trace[kTrMmaTotal] = clock64() - t_role0;
            p.trace[kTrMmaIssue] = tr[3];
        }
    } else if (warp < kFirstDrainWarp) {
        // ------------------------------------------------------------------ split
        // Two groups of four warps take alternate slabs, so that one slab's trip through registers (shared
        // memory -> split -> tensor memory, a few hundred cycles of latency) overlaps the next one's.  Ring
        // stages follow from the slab number; the stage counts are even, so a stage stays with one group.
        const int quarter = warp & 3;           // tensor-memory lane quarter this warp may access
        const int group = (warp - kFirstSplitWarp) >> 2;
        const int row = quarter * 32 + lane;    // token inside the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        static_assert(XS % kSplitGroups == 0 && AS % kSplitGroups == 0, "a ring stage must stay with one split-warp group");
        int slab0 = 0;  // slabs of this CTA's earlier tiles
        for (int tile = blockIdx.x; tile < n_tiles && !__any_sync(0xffffffffu, bad != 0); tile += tile_step) {
            const int nslabs = __ldg(p.group_slabs + tile % p.groups);
            // this group's slabs: s = group (mod kSplitGroups), counted over all tiles of the CTA
            for (int s = slab0 + (group + kSplitGroups - slab0 % kSplitGroups) % kSplitGroups; s < slab0 + nslabs; s += kSplitGroups) {
                const int xs = s % XS, as = s % AS;
                wait(x_full(xs), (uint32_t)(s / XS) & 1u, 0);
                // the test of the tensor-memory stage's release travels while the slab is read and split
                const uint32_t a_parity = ((uint32_t)(s / AS) & 1u) ^ 1u;
                const bool a_free = mbar_test_wait(a_empty(as), a_parity);
                const uint32_t a_hi = tmem_lane + C::kAccCols + as * C::kAStageCols;
                if (kIo16) {
                    // bf16 slab, 64-byte rows (64-byte swizzle: 16-byte chunk index XOR (row / 2) mod 4): the row's 32
                    // values are the 16 k-pairs tensor memory wants, as they lie
                    uint32_t packed[16];
                    const uint8_t* xrow = smem_gen + C::kOffX + xs * kSlabBytes + row * 64;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 v = *reinterpret_cast<const uint4*>(xrow + ((j ^ ((row >> 1) & 3)) << 4));
                        packed[4 * j + 0] = v.x; packed[4 * j + 1] = v.y; packed[4 * j + 2] = v.z; packed[4 * j + 3] = v.w;
                    }
                    if (!a_free) wait(a_empty(as), a_parity, 1);
                    tc_fence_after();
                    tmem_st16(a_hi, packed);
                } else {
                    uint32_t hi[32], lo[32];
                    {
                        const uint8_t* xrow = smem_gen + C::kOffX + xs * kSlabBytes + row * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            // 128-byte swizzle: the 16-byte chunk index is XORed with (row mod 8)
                            const uint4 v = *reinterpret_cast<const uint4*>(xrow + ((j ^ (row & 7)) << 4));
                            hi[j * 4 + 0] = v.x; hi[j * 4 + 1] = v.y; hi[j * 4 + 2] = v.z; hi[j * 4 + 3] = v.w;
                            if (kPasses == 3) {
                                tf32_lo_x2(v.x, v.y, lo[j * 4 + 0], lo[j * 4 + 1]);
                                tf32_lo_x2(v.z, v.w, lo[j * 4 + 2], lo[j * 4 + 3]);
                            }
                        }
                    }
                    if (!a_free) wait(a_empty(as), a_parity, 1);
                    tc_fence_after();
                    if (kPasses == 5) {
                        // columns 0-15: pairs of hi = bf16(x); columns 16-31: pairs of lo = bf16(x - hi)
                        uint32_t packed[32];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            split_bf16x2(__uint_as_float(hi[2 * j]), __uint_as_float(hi[2 * j + 1]), packed[j], packed[16 + j]);
                        }
                        tmem_st32(a_hi, packed);
                    } else if (kBf16) {
                        uint32_t packed[16];  // column j: k = 2j in the low half, k = 2j + 1 in the high half
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(hi[2 * j]), __uint_as_float(hi[2 * j + 1]));
                            packed[j] = *reinterpret_cast<const uint32_t*>(&pr);
                        }
                        tmem_st16(a_hi, packed);
                    } else {
                        tmem_st32(a_hi, hi);
                        if (kPasses == 3) tmem_st32(a_hi + 32, lo);
                    }
                }
                // The slab is released only here: the stores above took every loaded value as an operand, so the loads
                // have returned.  Released right after the loads were issued, the refill (TMA, async proxy) could
                // overtake reads still queued in the load/store unit (generic proxy); a proxy fence before the arrival
                // would also do, and costs 1-5 % more.
                mbar_arrive(x_empty(xs));
                tmem_wait_st();
                tc_fence_before();
                if ((lane == 0) & (bad == 0)) smem_add_release(a_count(as), 1u);  // nothing is published once a wait has given up
            }
            slab0 += nslabs;
        }
        if (tracing && warp == kFirstSplitWarp && lane == 0) {
            p.trace[kTrXfXFull] = tr[0];
            p.trace[kTrXfAEmpty] = tr[1];
            p.trace[kTrXfTotal] = clock64() - t_role0;
        }
    } else {
        // ------------------------------------------------------------------ drain (promotion + epilogue)
        const int quarter = warp & 3;          // tensor-memory lane quarter this warp may access
        const int row = quarter * 32 + lane;   // token inside the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        uint32_t ready_ph = 0;  // bit r: parity of the next p_ready[r] phase
        bool ok = true;
        int4 ahead = first_chunk();
        // Row-major output: a promotion goes through a staging tile in shared memory ([128 tokens][32 columns],
        // 128-byte swizzle) and leaves as ONE TMA store (the row's first promotion in the tile) or TMA
        // add-reduction (later ones) issued by one thread, instead of 16 scattered 16-byte loads and stores per
        // thread; rows beyond m are clipped by the tensor map.  Two staging tiles alternate.
        const bool issuer = warp == kFirstDrainWarp && lane == 0;
        uint32_t n_out = 0;          // promotions staged so far (selects the staging tile)
        // Returns false, to all four warps alike, when a thread of any of them has given up on a wait: the
        // first barrier carries that vote, so that the warps leave their loops together and none is left
        // behind at a barrier.
        // put_tile: the 128 threads' rows v go to the tile (col0, tok0) of the tensor behind `tmap`, overwriting it
        // or adding to it.
        auto put_tile = [&](const float (&v)[32], const CUtensorMap* tmap, int64_t col0, int32_t tok0, bool overwrite,
                            bool to_peers = false) -> bool {
            const uint32_t buf = smem_base + C::kOffOut + (n_out & 1u) * kSlabBytes;
            // the tile's previous store (two promotions ago) must have read it; a reduction additionally waits
            // until every earlier store of this thread is complete in global memory
            if (issuer) {
                if (!overwrite) bulk_wait_group<0>();
                else bulk_wait_group_read<1>();
            }
            uint32_t any_bad;
            asm volatile(
                "{\n\t.reg .pred q, r;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.or.pred r, 2, 128, q;\n\t"
                "selp.u32 %0, 1, 0, r;\n\t}"
                : "=r"(any_bad) : "r"(bad) : "memory");
            if (any_bad) return false;
            if (kIo16) {  // bf16 output tile: 64-byte rows under the 64-byte swizzle
                uint8_t* dst = smem_gen + C::kOffOut + (n_out & 1u) * kSlabBytes + row * 64;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t w[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const __nv_bfloat162 pr = __floats2bfloat162_rn(v[j * 8 + 2 * q], v[j * 8 + 2 * q + 1]);
                        w[q] = *reinterpret_cast<const uint32_t*>(&pr);
                    }
                    *reinterpret_cast<uint4*>(dst + ((j ^ ((row >> 1) & 3)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
                uint8_t* dst = smem_gen + C::kOffOut + (n_out & 1u) * kSlabBytes + row * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float4*>(dst + ((j ^ (row & 7)) << 4)) =
                        make_float4(v[j * 4 + 0], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
            }
            fence_proxy_async_smem();  // generic-proxy writes, read by the TMA through the async proxy
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (issuer) {
                if (to_peers && p.scatter_rows > 0) {
                    // reduce-scatter by rows: the completed tile goes to this rank's slot on the rank that owns its rows
                    const int32_t owner = (int32_t)(tok0 / p.scatter_rows);
                    const int32_t y = (int32_t)(p.scatter_slot * p.scatter_rows + (tok0 - owner * p.scatter_rows));
                    tma_store_2d(&peers.map[owner], buf, (int32_t)col0, y);
                } else {
                    if (overwrite) tma_store_2d(tmap, buf, (int32_t)col0, tok0);
                    else tma_reduce_add_2d(tmap, buf, (int32_t)col0, tok0);
                    if (to_peers)  // the completed tile also goes to every other GPU's copy of the output
                        for (int i = 0; i < p.n_peers; ++i) tma_store_2d(&peers.map[i], buf, (int32_t)col0, tok0);
                }
                bulk_commit_group();
            }
            ++n_out;
            return true;
        };
        auto gelu = [](float (&v)[32]) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
        };
        // One promotion of a row.  Without an activation the partial sums of a row simply add up in the output.
        // With one, they add up in the tensor that keeps the pre-activation values (pre_act if given, else the
        // output itself), and the row's last promotion produces the activated values from the completed sum --
        // directly when it is also the first (rows of up to kDrainEvery blocks: the usual case), else by adding
        // its part, waiting for that reduction, reading the total back and overwriting the output tile.
        auto stage_out = [&](float (&v)[32], int64_t col0, int32_t tok0, int64_t tok, bool live, bool first, bool last) -> bool {
            if (first) {
                if (p.bias != nullptr) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 add = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + j);
                        v[j * 4 + 0] += add.x; v[j * 4 + 1] += add.y; v[j * 4 + 2] += add.z; v[j * 4 + 3] += add.w;
                    }
                }
                if (p.residual != nullptr && live) {
                    const float4* res = reinterpret_cast<const float4*>(p.residual + tok * p.n + col0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 add = __ldg(res + j);
                        v[j * 4 + 0] += add.x; v[j * 4 + 1] += add.y; v[j * 4 + 2] += add.z; v[j * 4 + 3] += add.w;
                    }
                }
            }
            // x coordinate of the tile in the output tensor(s): the column slice this call owns starts at out_col0
            const int64_t xo = col0 + p.out_col0;
            if (p.act == 0 && p.n_peers == 0) return put_tile(v, &tmap_out, xo, tok0, first);
            // With an activation or peer outputs a tile leaves only when its row is complete.
            const bool keep_pre = p.pre_act != nullptr;
            const CUtensorMap* sums = keep_pre ? &tmap_pre : &tmap_out;
            const int64_t xs = keep_pre ? col0 : xo;
            if (!last) return put_tile(v, sums, xs, tok0, first);
            if (!first) {
                if (!put_tile(v, sums, xs, tok0, false)) return false;
                if (issuer) {
                    bulk_wait_group<0>();                              // the reduction has reached global memory
                    asm volatile("fence.proxy.async;" ::: "memory");   // async-proxy writes before the generic reads below
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                const float* total = keep_pre ? p.pre_act + tok * p.n + col0 : p.out + tok * p.out_ld + xo;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 t4 = live ? __ldcg(reinterpret_cast<const float4*>(total) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v[j * 4 + 0] = t4.x; v[j * 4 + 1] = t4.y; v[j * 4 + 2] = t4.z; v[j * 4 + 3] = t4.w;
                }
            } else if (keep_pre) {
                if (!put_tile(v, &tmap_pre, col0, tok0, true)) return false;
            }
            if (p.act != 0) gelu(v);
            return put_tile(v, &tmap_out, xo, tok0, true, true);
        };

        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += tile_step) {
            const int g = tile % p.groups;
            const int e0 = __ldg(p.group_off + g), e1 = __ldg(p.group_off + g + 1);
            const int nrows = min(G, p.n_out_blocks - g * G);
            const int32_t tok0 = (tile / p.groups) * kTileTokens;
            const int64_t tok = (int64_t)tok0 + row;
            const bool live = tok < p.m;

            // column-major output (the reference's buffer layout): direct stores
            // v (+ bias on a row's first promotion, + previous output afterwards) -> out[col0 .. col0+31][tok]
            auto emit_colmajor = [&](int r, const float (&v)[32], bool first) {
                if (!live) return;
                const int64_t col0 = ((int64_t)g * G + r) * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float* dst = p.out + (col0 + j) * p.m + tok;
                    float add = 0.f;
                    if (!first) add = *dst;
                    else if (p.bias != nullptr) add = __ldg(p.bias + col0 + j);
                    *dst = v[j] + add;
                }
            };
            auto emit = [&](int r, float (&v)[32], bool first, bool last) -> bool {
                if (p.out_colmajor) {
                    if (__any_sync(0xffffffffu, bad != 0)) return false;
                    emit_colmajor(r, v, first);
                    return true;
                }
                return stage_out(v, ((int64_t)g * G + r) * 32, tok0, tok, live, first, last);
            };

            uint32_t seen = 0;      // bit r: the row has been written once in this tile
            if (e0 == e1) ahead = skip_empty_tile(tile);
            for (int base = e0; base < e1 && ok; base += 32) {
                const int4 mine = ahead;
                ahead = prefetch(tile, base, e1);
                uint32_t drains = __ballot_sync(0xffffffffu, (mine.w & kDrainFlag) != 0);
                const uint32_t row_ends = __ballot_sync(0xffffffffu, (mine.w & kPlanRowEnd) != 0);
                while (drains != 0) {
                    const int i = __ffs(drains) - 1;
                    drains &= drains - 1;
                    const int r = __shfl_sync(0xffffffffu, mine.z, i);
                    wait(p_ready(r), (ready_ph >> r) & 1u, 0);  // (a wait that gave up is noticed in emit)
                    ready_ph ^= 1u << r;
                    tc_fence_after();
                    uint32_t main_[32];
                    float v[32];
                    tmem_ld32(tmem_lane + r * C::kRowCols, main_);
                    if (kSplit) {
                        uint32_t corr[32];
                        tmem_ld32(tmem_lane + r * C::kRowCols + 32, corr);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(main_[j]) + __uint_as_float(corr[j]);
                    } else {
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(main_[j]);
                    }
                    tc_fence_before();
                    mbar_arrive(p_taken(r));
                    ok = emit(r, v, !((seen >> r) & 1u), ((row_ends >> i) & 1u) != 0);
                    if (!ok) break;
                    seen |= 1u << r;
                }
            }
            if (ok) {
                // block-rows without any block: bias (+ residual, activated) or zero
                for (int r = 0; r < nrows && ok; ++r)
                    if (!((seen >> r) & 1u)) {
                        float z[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) z[j] = 0.f;
                        ok = emit(r, z, true, true);
                    }
            }
        }
        if (issuer) bulk_wait_group<0>();  // the staging tiles are read until the last store has finished
        if (tracing && warp == kFirstDrainWarp && lane == 0) {
            p.trace[kTrDrainPReady] = tr[0];
            p.trace[kTrDrainTotal] = clock64() - t_role0;
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

template <int G, int kPasses>
cudaError_t launch_dsd_g(const CUtensorMap& tmap_a, const CUtensorMap& tmap_out, const CUtensorMap& tmap_pre,
                         const PeerMaps& peers, const DsdParams& p, int64_t tiles, cudaStream_t stream) {
    // The shared-memory attribute and the SM count are per device: asked once per device and kernel variant,
    // then remembered (plain arrays; two threads racing on the first call store the same values).
    constexpr int kMaxDevices = 64;
    static int sm_count[kMaxDevices] = {0};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (sm_count[dev] == 0) {
        err = cudaFuncSetAttribute(dsd_umma_tf32_kernel<G, kPasses>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)Cfg<G, kPasses>::kSmemBytes);
        if (err != cudaSuccess) return err;
        int count = 0;
        err = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return err;
        sm_count[dev] = count;
    }
    const int sms = sm_count[dev];
    const int64_t n_tiles = (int64_t)p.groups * tiles;
    const unsigned grid = (unsigned)(n_tiles < sms ? n_tiles : sms);  // persistent: one CTA per SM
    dsd_umma_tf32_kernel<G, kPasses><<<grid, Cfg<G, kPasses>::kThreads, Cfg<G, kPasses>::kSmemBytes, stream>>>(tmap_a, tmap_out, tmap_pre, peers, p);
    return cudaGetLastError();
}

long long* g_trace_buffer = nullptr;  // host-side: device buffer the next dsd launches trace into
int g_trace_block = 0;

}  // namespace

void set_dsd_trace(long long* device_buffer, int block) {
    g_trace_buffer = device_buffer;
    g_trace_block = block;
}

cudaError_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                         uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return cudaErrorNotSupported;
    // The encoder is a driver entry point and wants a current context.  A thread that has made no runtime call
    // needing one yet (autograd's backward thread when the allocator serves everything from its cache) has none:
    // bind the runtime's context of the current device to it.
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaSetDevice(dev);
    if (err != cudaSuccess) return err;
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
                            bool out_colmajor, const DsdEpilogue& epilogue, cudaStream_t stream) {
    if (!is_umma_precision(precision)) return cudaErrorNotSupported;
    const bool io16 = epilogue.io_bf16;
    if (io16 && (precision != BSMM_PREC_BF16 || out_colmajor || epilogue.residual != nullptr || epilogue.pre_act != nullptr))
        return cudaErrorNotSupported;
    if (epilogue.n_peer_outs < 0 || epilogue.n_peer_outs > kMaxPeerOutputs) return cudaErrorInvalidValue;
    if (epilogue.scatter_rows != 0 &&
        (io16 || out_colmajor || epilogue.n_peer_outs == 0 || epilogue.scatter_rows < 0 ||
         (epilogue.scatter_rows % kTileTokens) != 0 || epilogue.scatter_rows * epilogue.n_peer_outs != m ||
         epilogue.scatter_slot < 0 || epilogue.scatter_slot >= epilogue.n_peer_outs))
        return cudaErrorInvalidValue;  // every token tile lies inside one owner's rows; the parts tensors are [m, out_ld] too
    const int64_t out_ld = epilogue.out_ld > 0 ? epilogue.out_ld : n;
    if (out_colmajor && (epilogue.n_peer_outs > 0 || out_ld != n || epilogue.out_col0 != 0)) return cudaErrorNotSupported;
    if (out_ld < n + epilogue.out_col0 || epilogue.out_col0 < 0 || (out_ld % 32) != 0 || (epilogue.out_col0 % 32) != 0)
        return cudaErrorInvalidValue;
    if (out_colmajor && (epilogue.residual != nullptr || epilogue.pre_act != nullptr || epilogue.activation != 0))
        return cudaErrorNotSupported;
    if (!plan_group_valid(group)) return cudaErrorInvalidValue;
    if (m == 0 || n == 0) return cudaSuccess;
    if (k == 0) return cudaErrorInvalidValue;  // nothing to contract over; a tensor map cannot describe it
    const int64_t n_out_blocks = n / 32;
    const int64_t groups = plan_groups(n_out_blocks, group);
    const int64_t tiles = (m + kTileTokens - 1) / kTileTokens;
    if (groups * tiles > 0x7fffffffll || m > 0x7fffffffll) return cudaErrorInvalidValue;

    // The box never exceeds the tensor: with fewer than 128 tokens the slab load fills only the first
    // m rows; the remaining accumulator lanes see stale values and their outputs are never stored.
    const uint32_t box_rows = (uint32_t)(m < kTileTokens ? m : kTileTokens);
    CUtensorMap tmap_a;
    cudaError_t err =
        io16 ? make_tmap_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, (uint64_t)k, (uint64_t)m, 32, box_rows,
                            CU_TENSOR_MAP_SWIZZLE_64B)
             : make_tmap_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a, (uint64_t)k, (uint64_t)m, 32, box_rows,
                            CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess) return err;
    // the epilogue's stores: boxes of 32 columns x up to 128 token rows of the row-major output
    CUtensorMap tmap_out = tmap_a;
    PeerMaps peers;
    for (int i = 0; i < kMaxPeerOutputs; ++i) peers.map[i] = tmap_a;  // placeholders where unused
    if (!out_colmajor) {
        auto out_map = [&](CUtensorMap* map, void* base) {
            return io16 ? make_tmap_2d(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, (uint64_t)out_ld, (uint64_t)m, 32, box_rows,
                                       CU_TENSOR_MAP_SWIZZLE_64B)
                        : make_tmap_2d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, (uint64_t)out_ld, (uint64_t)m, 32, box_rows,
                                       CU_TENSOR_MAP_SWIZZLE_128B);
        };
        err = out_map(&tmap_out, out);
        if (err != cudaSuccess) return err;
        for (int i = 0; i < epilogue.n_peer_outs; ++i) {
            if (epilogue.peer_outs[i] == nullptr) return cudaErrorInvalidValue;
            err = out_map(&peers.map[i], epilogue.peer_outs[i]);
            if (err != cudaSuccess) return err;
        }
    }

    CUtensorMap tmap_pre = tmap_out;
    if (epilogue.pre_act != nullptr) {
        err = make_tmap_2d(&tmap_pre, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, epilogue.pre_act, (uint64_t)n, (uint64_t)m, 32,
                           box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
        if (err != cudaSuccess) return err;
    }

    DsdParams p;
    p.residual = epilogue.residual;
    p.pre_act = epilogue.pre_act;
    p.act = epilogue.activation;
    p.n_peers = epilogue.n_peer_outs;
    p.out_ld = out_ld;
    p.out_col0 = epilogue.out_col0;
    p.scatter_rows = epilogue.scatter_rows;
    p.scatter_slot = epilogue.scatter_slot;
    p.packed = static_cast<const uint8_t*>(packed) + (dgrad ? nnz * packed_slot_bytes(precision) : 0);
    p.group_off = static_cast<const int32_t*>(plan);
    p.group_slabs = p.group_off + groups + 1;
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
    p.n_tiles = (int32_t)(groups * tiles);
    p.out_colmajor = out_colmajor ? 1 : 0;
    p.x_bytes = box_rows * (io16 ? 64u : 128u);
    p.trace = g_trace_buffer;
    p.trace_block = g_trace_block;
    const bool split = precision == BSMM_PREC_TF32X3;
    if (is_split_precision(precision) && group == 8) return cudaErrorInvalidValue;  // 8 rows x 64 columns leave no tensor memory for A
    if (precision == BSMM_PREC_BF16X3) {
        switch (group) {
            case 4: return launch_dsd_g<4, 5>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
            case 6: return launch_dsd_g<6, 5>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    if (precision == BSMM_PREC_BF16) {
        if (group == 5) return cudaErrorInvalidValue;  // the 5-row tile exists for 3xTF32 only
        if (io16) {
            switch (group) {
                case 4: return launch_dsd_g<4, 4>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
                case 6: return launch_dsd_g<6, 4>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
                default: return launch_dsd_g<8, 4>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
            }
        }
        switch (group) {
            case 4: return launch_dsd_g<4, 0>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
            case 6: return launch_dsd_g<6, 0>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
            default: return launch_dsd_g<8, 0>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
        }
    }
    if (group == 5) return split ? launch_dsd_g<5, 3>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream) : cudaErrorInvalidValue;
    switch (group) {
        case 4: return split ? launch_dsd_g<4, 3>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream) : launch_dsd_g<4, 1>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
        case 6: return split ? launch_dsd_g<6, 3>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream) : launch_dsd_g<6, 1>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
        default: return launch_dsd_g<8, 1>(tmap_a, tmap_out, tmap_pre, peers, p, tiles, stream);
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

}  // namespace bsmm
