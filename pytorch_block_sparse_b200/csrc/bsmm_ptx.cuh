// Inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA (tensor and
// linear bulk copies), tensor memory (tcgen05.alloc/ld/st) and the tcgen05 MMA.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bsmm {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of the (converged) warp is elected; the warp's control flow stays uniform, so the operands
// of the single-thread instructions issued under it (TMA, tcgen05.mma, tcgen05.commit) can live in
// uniform registers instead of being moved there lane by lane.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// A counter in shared memory as a publication flag: writers add with release semantics, readers poll with
// acquire semantics.  Unlike a phase-parity barrier it cannot be misread by a waiter that skipped phases.
__device__ __forceinline__ void smem_add_release(uint32_t addr, uint32_t value) {
    asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t smem_load_acquire(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// Non-blocking test of the same condition (try_wait may suspend the warp for a while when the phase is open).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// How many consecutive stages of a ring of `stages` barriers (8 bytes apart from `bar0`) have completed
// their awaited phase, starting with stage `stage` whose awaited parity is `parity` (stages that wrap around
// await the other parity).  One barrier per lane in a single instruction: a successful wait costs about 85
// cycles of latency whether it tests one barrier or thirty-two, so a warp that consumes stages one by one
// looks ahead with this and then skips the waits it already knows the answer to.  All lanes must call it.
__device__ __forceinline__ int mbar_ring_ready(uint32_t bar0, int stages, int stage, uint32_t parity, int lane) {
    int st = stage + lane;
    uint32_t par = parity;
    if (st >= stages) { st -= stages; par ^= 1u; }
    const bool ok = lane < stages && mbar_test_wait(bar0 + 8u * (uint32_t)st, par);
    const uint32_t mask = __ballot_sync(0xffffffffu, ok);
    return __ffs(~mask) - 1;
}

// Bounded wait.  Gives up after ~2^31 SM cycles (about a second) or as soon as another thread of
// the CTA has given up (`*abort_flag` != 0); on giving up it raises the flag itself.
// Returns true when the phase completed.
constexpr long long kWaitCycles = 1ll << 31;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0) return false;
        if (clock64() - t0 > kWaitCycles) {
            *abort_flag = 1;
            return false;
        }
    }
}

// lo parts of the 3xTF32 splitting of two fp32 values (bit patterns): x - trunc_tf32(x), the two subtractions as
// one packed instruction.
__device__ __forceinline__ void tf32_lo_x2(uint32_t x0, uint32_t x1, uint32_t& lo0, uint32_t& lo1) {
    asm("{\n\t.reg .b64 a, t, d;\n\t"
        "mov.b64 a, {%2, %3};\n\t"
        "mov.b64 t, {%4, %5};\n\t"
        "sub.rn.f32x2 d, a, t;\n\t"
        "mov.b64 {%0, %1}, d;\n\t}"
        : "=r"(lo0), "=r"(lo1)
        : "r"(x0), "r"(x1), "r"(x0 & 0xffffe000u), "r"(x1 & 0xffffe000u));
}

// Two-part bf16 splitting of a pair of fp32 values: hi = {bf16(x0), bf16(x1)} (round to nearest, x0 in the low
// half), lo = {bf16(x0 - hi0), bf16(x1 - hi1)}.  The differences are exact in fp32; the mixed-precision fma takes
// the bf16 halves of hi as they are (hi * -1 + x), so nothing is unpacked: four instructions per pair.
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    asm("{\n\t.reg .b16 h0, h1, m1;\n\t.reg .f32 d0, d1;\n\t"
        "cvt.rn.bf16x2.f32 %0, %3, %2;\n\t"
        "mov.b32 {h0, h1}, %0;\n\t"
        "mov.b16 m1, 0xBF80;\n\t"
        "fma.rn.f32.bf16 d0, h0, m1, %2;\n\t"
        "fma.rn.f32.bf16 d1, h1, m1, %3;\n\t"
        "cvt.rn.bf16x2.f32 %1, d1, d0;\n\t}"
        : "=&r"(hi), "=r"(lo)
        : "f"(x0), "f"(x1));
}

// ---------------------------------------------------------------- TMA
// 2-D tiled load: box starting at element (x, y) of the tensor described by `tmap` -> smem,
// completing `bar` with the box's byte count.  x * element size must be a multiple of 16 B.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int32_t x, int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// 2-D tiled store smem -> global (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
// 2-D tiled reduction smem -> global: global += smem, element type from the tensor map.
__device__ __forceinline__ void tma_reduce_add_2d(const void* tmap, uint32_t src, int32_t x, int32_t y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Linear bulk copy global -> smem; both addresses 16-B aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 columns of 32-bit: thread i of the warp <-> lane (base lane + i), register j <-> column (base + j).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---------------------------------------------------------------- tcgen05 MMA
// Shared-memory operand descriptor, un-swizzled canonical layout: 14-bit fields in 16-B units
// (start address, leading-dimension byte offset, stride-dimension byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_noswizzle(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46);
}
// Same with the 128-byte swizzle mode (layout type 2 in bits 61..63).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return smem_desc_noswizzle(addr, lbo_bytes, sbo_bytes) | (2ull << 61);
}
// Same with the "128-byte swizzle, 32-byte atomicity" mode (layout type 1), the only layout the tensor
// core accepts for MN-major operands of 32-bit element types; TMA writes it with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  Its swizzle atom is 4 k-rows of 128 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128_base32(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return smem_desc_noswizzle(addr, lbo_bytes, sbo_bytes) | (1ull << 61);
}
// Same with the 64-byte swizzle mode (layout type 4).
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return smem_desc_noswizzle(addr, lbo_bytes, sbo_bytes) | (4ull << 61);
}
// Instruction descriptor, fp32 accumulate.  fmt: 0 f16, 1 bf16, 2 tf32.  *_mn_major: operand is
// MN-major (its M/N index is the contiguous one) instead of K-major.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t m, uint32_t n, bool a_mn_major,
                                                   bool b_mn_major) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]   (A K-major in tensor memory: lane = row, column = k)
__device__ __forceinline__ void mma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ss_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrive once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t tf32_rna_bits(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

}  // namespace ptx
}  // namespace bsmm
