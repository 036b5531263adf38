// Blackwell (sm_100a) building blocks in inline PTX: mbarrier with bounded waits, TMA tile loads,
// tensor-memory allocation, tcgen05.mma issue/commit and tcgen05.ld.  No multicast forms are used
// anywhere: every CTA loads its own operand tiles, so the same kernels are safe under tensor
// parallelism when an operand lives in peer memory.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "ps_common.cuh"

namespace ps {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait: gives up after ~`budget` clock cycles and returns false; the caller records
// PS_DEV_WAIT_TIMEOUT and unwinds (frees tensor memory, stops issuing) instead of spinning forever.
// Launchers pass the library-wide budget (g_ps_wait_budget_cycles); the constant is only a default.
constexpr long long kWaitBudgetCycles = 2000000000ll;   // about one second at B200 clocks
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long budget = kWaitBudgetCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > budget) return false;
    }
    return true;
}

// Bounded wait with a caller-chosen budget that also gives up as soon as another role of the CTA has
// raised `abort_flag` (so one timed-out role unwinds the whole CTA quickly).  On expiry it raises the
// flag itself.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, long long budget,
                                                    volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 31) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > budget) { *abort_flag = 1; return false; }
        }
    }
    return true;
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// 2-D tiled TMA load (no multicast).  Coordinates are (innermost, outer) element indices; the
// innermost coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// L2 prefetches (no shared memory, no completion tracking): a 2-D tile through a tensor map, and a plain byte range
// (16-byte aligned address, size a multiple of 16).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 64 bf16 x rows with CU_TENSOR_MAP_SWIZZLE_128B produces):
// 8-row groups are 1024 bytes apart (SBO), LBO is unused for swizzled K-major layouts.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                     // leading byte offset (ignored)
    d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset
    d |= (uint64_t)1 << 46;                     // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16, A/B = bf16 K-major, D = fp32.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- block-scaled MMA (kind::mxf4nvf4 / kind::mxf8f6f4.block_scale)
//
// Scale factors live in tensor memory.  For an operand tile of R rows (R = 128 for the M side, the N
// extent for the N side) the factors of row r sit in lane r % 32 (replicated into all four 32-lane
// sub-partitions), 32-bit column r / 32, and the four bytes of that word are four consecutive
// K-blocks.  The shared-memory image of one such "atom" (128 rows x 4 factors = 512 bytes) is
//     byte (r % 32) * 16 + (r / 32) * 4 + j        (j = K-block 0..3)
// which `tcgen05.cp.32x128b.warpx4` moves into four tensor-memory columns in one instruction.
// NVFP4 (16-element blocks, UE4M3): one atom per 64-element MMA, all four bytes used.
// MXFP8 (32-element blocks, UE8M0): one atom per four 32-element MMAs, byte selected by the
// instruction descriptor's scale-factor id.
constexpr uint32_t kSfAtomBytes = 512;

// Matrix descriptor of a scale-factor atom for tcgen05.cp: no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(128 >> 4) << 32;            // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                     // descriptor version (Blackwell)
    return d;                                   // layout type 0 = no swizzle, leading offset unused
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Operand formats of the block-scaled kinds.
constexpr uint32_t kFmtE4M3 = 0, kFmtE2M1_mxf4 = 1;
constexpr uint32_t kSfUE4M3 = 0, kSfUE8M0 = 1;
// Instruction descriptor for block-scaled MMA: A and B K-major, fp32 accumulate.
__host__ __device__ constexpr uint32_t idesc_block_scaled(int M, int N, uint32_t ab_format, uint32_t sf_format,
                                                          uint32_t a_sf_id, uint32_t b_sf_id) {
    return (b_sf_id << 4) | (ab_format << 7) | (ab_format << 10) | ((uint32_t)(N >> 3) << 17) | (sf_format << 23) |
           ((uint32_t)(M >> 4) << 24) | (a_sf_id << 29);
}
// D[tmem] (+)= A[smem] . B[smem]^T, E2M1 operands with one UE4M3 scale per 16 elements; K = 64.
__device__ __forceinline__ void mma_nvfp4_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
// Same with E4M3 operands and one UE8M0 scale per 32 elements; K = 32.
__device__ __forceinline__ void mma_mxfp8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

// Registers -> tensor memory: thread i of the warp writes lane (lane base + i), 4 (or 1) consecutive columns.
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tmem_st_32x1(uint32_t taddr, uint32_t a) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(a) : "memory");
}
// Sixteen consecutive columns in one instruction; columns 0, 4, 8, 12 take a, b, c, d, the rest a filler.
__device__ __forceinline__ void tmem_st_32x16_sparse4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %5, %5, %5, %2, %5, %5, %5, %3, %5, %5, %5, %4, %5, %5, %5};"
                 ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(0u) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 64-bit descriptor from two 32-bit halves (lets callers keep the constant half out of the inner loop).
__device__ __forceinline__ uint64_t desc_pack(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
// Halves of smem_desc_sw128 / smem_desc_sf: low word = (address >> 4) [| LBO field], high word constant.
constexpr uint32_t kDescSw128Hi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescSw128LoFlags = 1u << 16;
constexpr uint32_t kDescSfHi = (uint32_t)(128 >> 4) | (1u << 14);

// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tc
}  // namespace ps
