// Causal paged attention for prefill-sized steps on the fifth-generation tensor cores (head dim 256, bf16 pools,
// pages of 16, 32 or 64 tokens): one CTA = 128 consecutive query rows of one sequence and one query head.
//
//   warp 8   TMA producer for Q (once) and the K tiles: a 64-token tile is four pages, each fetched as four
//            64-column boxes (128-byte swizzle) straight from the paged pool through a tensor map over
//            [pages * kv heads * page tokens, D] (one, two or four pages per tile for 64-, 32-, 16-token pages); two stages.
//   warp 9   TMA producer for the V tiles (same boxes, two stages).
//   warps 10, 11  one thread each issues S(t) = Q K(t)^T (tcgen05.mma, 16 products of 128 x 64 x 16) into one of two
//            64-column accumulators, warp 10 for even t and warp 11 for odd t, as soon as the K stage and the
//            accumulator are free, so the tensor core computes the next scores while the softmax warps work on
//            the current ones.
//   warp 12  one thread issues O += P(t) V(t) into a 256-column accumulator.  V is consumed as it lies in the
//            pool (token rows, dims contiguous): an MN-major B operand.
//   warps 0-7  softmax: two threads own a query row (= TMEM lane), 32 score columns each.  Scores come back with
//            tcgen05.ld (both threads read the whole row for its maximum: no shuffles, no exchange), probabilities go
//            to shared memory as a bf16 K-major A operand (swizzled by hand), and the output accumulator is
//            rescaled in tensor memory only when a row's maximum has grown
//            by more than 2^8 since the reference used for its exponents (the sum absorbs the difference, so the
//            result is the exact softmax).  The epilogue normalises, applies the sigmoid output gate and writes
//            bf16 through shared memory with coalesced 16-byte stores.
//
// Every wait is bounded; a timeout raises the CTA's abort flag, every role unwinds, outstanding copies get a
// bounded chance to land, tensor memory is freed and PS_DEV_WAIT_TIMEOUT is recorded.  Token rows of the last
// tile that lie beyond the sequence's end are zeroed in shared memory before the P V product (their
// probabilities are zero, but stale pool contents must not be able to inject NaNs).
//
// The reference's prefill attention (src/phaseshift/models/qwen35/kernels/optimized/attention/
// paged_prefill.hip:408-874) tiles 16 query rows per wave on WMMA; FP8 pools, other head sizes and other page
// sizes stay on the mma.sync kernel (attn_prefill.cu).
#include <cuda.h>

#include "ps_common.cuh"
#include "ps_tcgen05.cuh"

namespace ps {

constexpr int kTcRows = 128, kTcTok = 64, kTcD = 256;
constexpr int kTcThreads = 416;                      // warps 0-7 softmax, 8 Q / K producer, 9 V producer, 10-11 S issuers, 12 P V issuer
constexpr int kTcQBytes = kTcRows * kTcD * 2;         // 64 KB: four 64-column boxes of 128 rows
constexpr int kTcKvStage = kTcTok * kTcD * 2;         // 32 KB: four 64-column boxes of 64 tokens
constexpr int kTcPBuf = kTcRows * kTcTok * 2;         // 16 KB: 128 rows x 64 tokens
constexpr int kTcSmem = kTcQBytes + 4 * kTcKvStage + 2 * kTcPBuf;
constexpr int kTcOutPitch = kTcD + 8;                 // staging pitch of the epilogue (elements)
constexpr uint32_t kTcTmemCols = 512;                 // S0 | S1 (64 each) | O (256)

struct AttnTcArgs {
    const int* block_table; int max_blocks; int num_pages; int page_tokens;     // page_tokens: 16, 32 or 64
    const int* seqs;             // [n_seqs][4] = row_start, n_rows, slot, pos_start
    int Hq, Hkv; float scale_log2;
    int min_rows;                // sequences with at most this many rows in the step are left to the split-KV kernel
    const __nv_bfloat16* gate; int ld_gate; int gate_head_stride; int gate_offset;
    __nv_bfloat16* out;          // [rows, Hq * D]
    uint32_t* status;
    long long budget;
    // decode / verify variant (DEC): split-KV partials in the layout of the per-row kernel's merge pass
    int split_tokens; int max_splits; int dec_max_rows;
    float* part_acc; float* part_ml;
    long long* prof;             // optional cycle stamps of CTA (0, 0, 0): [32 tiles][16], softmax slots 0-7, issuer slots 8-12
};

namespace tc {
// Shared-memory descriptor of an MN-major operand (rows = K index, 128 bytes = 64 MN elements per row, 128-byte
// swizzle): `lbo` bytes between 64-element groups along MN, `sbo` bytes between 8-row groups along K.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, A = bf16 K-major, B = bf16 MN-major, D = fp32.
__host__ __device__ constexpr uint32_t idesc_bf16_f32_bmn(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
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
}  // namespace tc

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// sigmoid(x) = 0.5 + 0.5 tanh(x / 2) with the hardware tanh (one special-function operation instead of an exponential and a
// reciprocal; absolute error about 5e-4, a fraction of the bf16 rounding step of the gated output).  A full-precision
// division here made the epilogue the longest phase of a short CTA.
__device__ __forceinline__ float sigmoid_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}

// Prefill (DEC = false): grid = (q tiles of 128 rows, Hq, n_seqs); the heaviest (latest) query tiles are scheduled first.
// Decode / verify (DEC = true): grid = (KV splits, Hkv, n_seqs).  A CTA serves one sequence with at most 16 rows in the step
// and one KV head: tile row 8 r + g is query head g of that KV head for the sequence's row r (grouped-query packing: the G <= 8
// heads that share the KV head ride in one MMA tile, so K and V are read once for all of them), over the tokens of its
// split; it leaves unnormalised partial outputs and (maximum, sum) pairs for the merge pass of paged_attention.cu.
template <bool DEC>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const AttnTcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // Q, two K and two V stages, two P buffers: 224 KB, which with the static part below is the whole 227 KB of the SM;
    // the swizzled tiles need the 1024-byte alignment that the declaration asks for (checked, not assumed)
    unsigned char* smem = smem_raw;
    if ((tc::smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) set_status(a.status, PS_DEV_BAD_INDEX);
        return;
    }
    unsigned char* sQ = smem;
    unsigned char* sK = sQ + kTcQBytes;
    unsigned char* sV = sK + 2 * kTcKvStage;
    unsigned char* sP = sV + 2 * kTcKvStage;
    __shared__ __align__(8) uint64_t q_full, k_full[2], v_full[2], s_full[2], p_full[2], pv_done[2];
    __shared__ float s_l[2][kTcRows];            // row sums of the two column halves, exchanged once at the end
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_abort, s_bad, k_issued, k_consumed, v_issued, v_consumed, q_issued, q_consumed;

    const int* sd = a.seqs + 4 * blockIdx.z;
    const int row_start = sd[0], n_rows = sd[1], slot = sd[2], pos_start = sd[3];
    const int G = a.Hq / a.Hkv;
    int r_begin, nq, h, kvh, pos_q0, kv_end, t_first, T;
    if constexpr (DEC) {
        if (slot < 0 || n_rows <= 0 || n_rows > a.dec_max_rows) return;
        r_begin = 0; nq = 8 * n_rows; kvh = blockIdx.y; h = kvh * G;
        pos_q0 = pos_start; kv_end = pos_start + n_rows;
        const int tps = a.split_tokens / kTcTok;                         // tiles per split
        t_first = (int)blockIdx.x * tps;
        const int t_end = min((kv_end + kTcTok - 1) / kTcTok, t_first + tps);
        if (t_first >= t_end) return;
        T = t_end - t_first;
    } else {
        const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;
        r_begin = tile * kTcRows;
        if (r_begin >= n_rows || slot < 0 || n_rows <= a.min_rows) return;
        nq = min(kTcRows, n_rows - r_begin);
        h = blockIdx.y; kvh = h / G;
        pos_q0 = pos_start + r_begin;
        kv_end = pos_q0 + nq;
        t_first = 0;
        T = (kv_end + kTcTok - 1) / kTcTok;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool cta_stamp = a.prof != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    if (cta_stamp) a.prof[15] = clock64();

    if (threadIdx.x == 0) {
        tc::mbar_init(&q_full, 1);
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(&k_full[s], 1); tc::mbar_init(&v_full[s], 1); tc::mbar_init(&s_full[s], 1);
            tc::mbar_init(&p_full[s], 8); tc::mbar_init(&pv_done[s], 1);
        }
        tc::fence_barrier_init();
        s_abort = 0; s_bad = 0; k_issued = k_consumed = v_issued = v_consumed = q_issued = q_consumed = 0;
        tc::tma_prefetch_desc(&map_q); tc::tma_prefetch_desc(&map_k); tc::tma_prefetch_desc(&map_v);
    }
    if (warp == 12) {
        tc::tmem_alloc(&tmem_base_slot, kTcTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_slot;
    const uint32_t tmem_o = tmem + 128;

    if (warp == 8 || warp == 9) {
        // ------------------------------------------------ TMA producers: warp 8 = Q and K, warp 9 = V.  One lane per box (a
        // tile is up to 16 boxes: pages x four 64-column groups): issuing them from one thread one after the other costs
        // more than a thousand cycles, and the stage's consumer is waiting for them.
        const bool isK = warp == 8;
        if (isK) {
            if constexpr (DEC) {
                // one 8-row box per (row of the sequence, 64-column group): the G heads of this KV head are consecutive rows
                // of the [rows * Hq, D] view of q; tile rows 8 r + g with g >= G hold other heads' values and are never used
                if (lane == 0) tc::mbar_expect_tx(&q_full, (uint32_t)n_rows * 4u * 1024u);
                __syncwarp();
                for (int i = lane; i < 4 * n_rows; i += 32) {
                    const int r = i >> 2, c4 = i & 3;
                    tc::tma_load_2d(sQ + c4 * (kTcRows * 128) + (8 * r) * 128, &map_q, c4 * 64, (row_start + r) * a.Hq + h, &q_full);
                }
            } else {
                if (lane == 0) tc::mbar_expect_tx(&q_full, kTcQBytes);
                __syncwarp();
                if (lane < 4) tc::tma_load_2d(sQ + lane * (kTcRows * 128), &map_q, h * kTcD + lane * 64, row_start + r_begin, &q_full);
            }
            if (lane == 0) q_issued = 1;
        }
        const int* bt = a.block_table + (size_t)slot * a.max_blocks;
        const int pt = a.page_tokens, ppt = kTcTok / pt;            // a page is one box of pt token rows per 64-column group
        const int pg = lane >> 2, cb = lane & 3;
        const bool active = pg < ppt;
        unsigned char* stage0 = isK ? sK : sV;
        uint64_t* full = isK ? k_full : v_full;
        uint64_t* freed = isK ? s_full : pv_done;                   // a K stage is free once S(t) has read it, a V stage after P V(t)
        const CUtensorMap* map = isK ? &map_k : &map_v;
        for (int t = 0; t < T; ++t) {
            const int b = t & 1;
            int page = 0;
            const int blk = (t_first + t) * ppt + pg;
            if (active && blk * pt < kv_end) {
                page = bt[blk];
                if (page < 0 || page >= a.num_pages) { s_bad = 1; page = 0; }
            }
            if (t >= 2 && !__all_sync(0xffffffffu, tc::mbar_wait_abortable(&freed[b], (uint32_t)((t - 2) >> 1) & 1u, a.budget, &s_abort))) break;
            if (lane == 0) tc::mbar_expect_tx(&full[b], kTcKvStage);
            __syncwarp();
            if (active)
                tc::tma_load_2d(stage0 + b * kTcKvStage + cb * (kTcTok * 128) + pg * (pt * 128), map, cb * 64, (page * a.Hkv + kvh) * pt, &full[b]);
            if (lane == 0) { if (isK) k_issued = t + 1; else v_issued = t + 1; }
        }
    } else if (warp == 10 || warp == 11) {
        // ------------------------------------------------ score issuers: warp 10 issues S(t) for even t, warp 11 for odd t.
        // A tcgen05.mma costs its issuing thread about 80 cycles whatever its size, and a 128 x 64 x 16 product is only 32
        // cycles of tensor work, so one thread cannot keep the pipe fed; two threads take turns.
        if (lane == 0) {
            constexpr uint32_t idesc_s = tc::idesc_bf16_f32(kTcRows, kTcTok);
            const int b = warp - 10;
            const uint32_t q_addr = tc::smem_u32(sQ), k_addr = tc::smem_u32(sK) + b * kTcKvStage;
            bool ok = tc::mbar_wait_abortable(&q_full, 0, a.budget, &s_abort);
            if (ok) q_consumed = 1;
            for (int t = b; t < T && ok; t += 2) {
                const uint32_t ph = (uint32_t)(t >> 1) & 1u;
                const bool stamp = a.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && t < 32;
                if (stamp) a.prof[t * 16 + 8] = clock64();
                // the score buffer is free once the softmax warps have read S(t - 2), which they signal with P(t - 2)
                if (t >= 2 && !tc::mbar_wait_abortable(&p_full[b], ph ^ 1u, a.budget, &s_abort)) { ok = false; break; }
                if (!tc::mbar_wait_abortable(&k_full[b], ph, a.budget, &s_abort)) { ok = false; break; }
                if (stamp) a.prof[t * 16 + 9] = clock64();
                atomicMax(&k_consumed, t + 1);
                tc::fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < kTcD / 16; ++ks) {
                    const uint64_t adesc = tc::smem_desc_sw128(q_addr + (ks >> 2) * (kTcRows * 128) + (ks & 3) * 32);
                    const uint64_t bdesc = tc::smem_desc_sw128(k_addr + (ks >> 2) * (kTcTok * 128) + (ks & 3) * 32);
                    tc::mma_bf16_ss(tmem + b * kTcTok, adesc, bdesc, idesc_s, ks > 0 ? 1u : 0u);
                }
                tc::mma_commit(&s_full[b]);
                if (stamp) a.prof[t * 16 + 10] = clock64();
            }
        }
    } else if (warp == 12) {
        // ------------------------------------------------ output issuer: O += P(t) V(t)
        if (lane == 0) {
            constexpr uint32_t idesc_o = tc::idesc_bf16_f32_bmn(kTcRows, kTcD);
            const uint32_t v_addr = tc::smem_u32(sV), p_addr = tc::smem_u32(sP);
            for (int t = 0; t < T; ++t) {
                const int b = t & 1;
                const uint32_t ph = (uint32_t)(t >> 1) & 1u;
                const bool stamp = a.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && t < 32;
                if (!tc::mbar_wait_abortable(&p_full[b], ph, a.budget, &s_abort)) break;
                if (stamp) a.prof[t * 16 + 11] = clock64();
                if (!tc::mbar_wait_abortable(&v_full[b], ph, a.budget, &s_abort)) break;
                v_consumed = t + 1;
                tc::fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kTcTok / 16; ++kk) {
                    const uint64_t adesc = tc::smem_desc_sw128(p_addr + b * kTcPBuf + kk * 32);
                    const uint64_t bdesc = tc::smem_desc_sw128_mn(v_addr + b * kTcKvStage + kk * (16 * 128), kTcTok * 128, 1024);
                    tc::mma_bf16_ss(tmem_o, adesc, bdesc, idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
                }
                tc::mma_commit(&pv_done[b]);
                if (stamp) a.prof[t * 16 + 12] = clock64();
            }
        }
    } else {
        // ------------------------------------------------ softmax warps 0-7: two threads per query row.  Warp w works on
        // TMEM lanes 32 (w % 4) .. + 31 (the quadrant a warp may touch) and on score columns 32 (w / 4) .. + 31 of the tile.
        const int quad = warp & 3, half = warp >> 2;
        const int row = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const int rp = DEC ? pos_q0 + (row >> 3) : pos_q0 + row;     // position of this thread's query row
        const float sc = a.scale_log2;
        float m_ref = 0.f, l_run = 0.f;
        bool ok = true;
        // the epilogue reads this tile's gate values (one 512-byte run per row): ask for them now, so that they come from
        // L2 then
        if (!DEC && a.gate != nullptr && half == 0 && row < nq)
            tc::bulk_prefetch_l2(a.gate + (size_t)(row_start + r_begin + row) * a.ld_gate + (size_t)h * a.gate_head_stride + a.gate_offset, kTcD * 2);
        for (int t = 0; t < T; ++t) {
            const int b = t & 1;
            const uint32_t ph = (uint32_t)(t >> 1) & 1u;
            const int tt = t_first + t;                               // tile index within the sequence
            const int t0 = tt * kTcTok + half * 32;                   // first token of this thread's columns
            const bool stamp = a.prof != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && t < 32;
            if (stamp) a.prof[t * 16 + 0] = clock64();
            ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(&s_full[b], ph, a.budget, &s_abort));
            if (!ok) break;
            tc::fence_after_sync();
            if (stamp) a.prof[t * 16 + 1] = clock64();
            // both threads of a row read all 64 scores and take the maximum themselves (cheaper than an exchange through
            // shared memory); each then exponentiates its own 32 columns
            uint32_t sr[32], so[32];
            tc::tmem_ld_32x32(tmem + lane_base + b * kTcTok + half * 32, sr);
            tc::tmem_ld_32x32(tmem + lane_base + b * kTcTok + (half ^ 1) * 32, so);
            tc::tmem_ld_wait();
            if (stamp) a.prof[t * 16 + 2] = clock64();
            if (tt * kTcTok + kTcTok - 1 > pos_q0) {                  // some row of the tile does not see every token
                const int to = tt * kTcTok + (half ^ 1) * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (t0 + j > rp) sr[j] = 0xff800000u;             // -inf
                    if (to + j > rp) so[j] = 0xff800000u;
                }
            }
            float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 32; ++j) mq[j & 3] = fmaxf(mq[j & 3], fmaxf(__uint_as_float(sr[j]), __uint_as_float(so[j])));
            float mx = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])) * sc;     // scale > 0, so the maximum commutes with it
            if (stamp) a.prof[t * 16 + 3] = clock64();
            float alpha = 1.f;
            if (t == 0) m_ref = mx == -INFINITY ? 0.f : mx;           // (a row that sees nothing here keeps a finite reference)
            else if (mx > m_ref + 8.f) { alpha = ex2_approx(m_ref - mx); m_ref = mx; }
            const bool rescale = __any_sync(0xffffffffu, alpha != 1.f);
            float sq[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const float p0 = ex2_approx(fmaf(__uint_as_float(sr[j]), sc, -m_ref));
                const float p1 = ex2_approx(fmaf(__uint_as_float(sr[j + 1]), sc, -m_ref));
                sq[(j >> 1) & 3] += p0 + p1;
                pk[j >> 1] = f32x2_to_bf16x2_bits(p0, p1);
            }
            l_run = l_run * alpha + ((sq[0] + sq[1]) + (sq[2] + sq[3]));
            if (t >= 2) {                                             // P buffer b was read by P V(t - 2)
                ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(&pv_done[b], (uint32_t)((t - 2) >> 1) & 1u, a.budget, &s_abort));
                if (!ok) break;
            }
            if (stamp) a.prof[t * 16 + 4] = clock64();
            unsigned char* prow = sP + b * kTcPBuf + row * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(prow + (((half * 4 + c) ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            if (t == T - 1 && kv_end < (tt + 1) * kTcTok) {
                // token rows of the last V tile beyond the sequence's end: zero them (whole 128-byte rows, so the swizzle
                // does not matter)
                ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(&v_full[b], ph, a.budget, &s_abort));
                if (!ok) break;
                const int jz = kv_end - tt * kTcTok;
                unsigned char* vs = sV + b * kTcKvStage;
                for (int i = (int)threadIdx.x; i < (kTcTok - jz) * 32; i += 2 * kTcRows) {
                    const int r = jz + (i >> 5), cb = (i & 31) >> 3, c = i & 7;
                    *reinterpret_cast<uint4*>(vs + cb * (kTcTok * 128) + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            if (stamp) a.prof[t * 16 + 5] = clock64();
            tc::fence_proxy_async_smem();
            if (stamp) a.prof[t * 16 + 6] = clock64();
            if (rescale) {                                            // t >= 1: O must be complete up to P V(t - 1)
                ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(&pv_done[b ^ 1], (uint32_t)((t - 1) >> 1) & 1u, a.budget, &s_abort));
                if (!ok) break;
                tc::fence_after_sync();
#pragma unroll 1
                for (int c0 = half * (kTcD / 2); c0 < (half + 1) * (kTcD / 2); c0 += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(tmem_o + lane_base + c0, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                    tc::tmem_st_32x32(tmem_o + lane_base + c0, r);
                }
                tc::tmem_st_wait();
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&p_full[b]);
            if (stamp) a.prof[t * 16 + 7] = clock64();
        }
        // ---- epilogue: O / l -> bf16 rows staged in shared memory (Q and K stages are free once the last P V is done)
        if (ok) ok = __all_sync(0xffffffffu, tc::mbar_wait_abortable(&pv_done[(T - 1) & 1], (uint32_t)((T - 1) >> 1) & 1u, a.budget, &s_abort));
        if (cta_stamp) a.prof[2 * 16 + 15] = clock64();
        s_l[half][row] = l_run;
        asm volatile("bar.sync 1, 256;" ::: "memory");               // the eight softmax warps only; every one of them gets here
        if (cta_stamp) a.prof[3 * 16 + 15] = clock64();
        if constexpr (DEC) {
            // partial result of this split for query row (r, g): unnormalised output, reference maximum (natural-log units, as
            // the merge pass expects) and sum
            const int r = row >> 3, g = row & 7;
            const bool mine = row < nq && g < G;
            if (ok && quad * 32 < nq) {                              // warp-uniform: the tensor-memory loads are collective
                tc::fence_after_sync();
                const size_t idx = ((size_t)(row_start + (mine ? r : 0)) * a.Hq + h + (mine ? g : 0)) * a.max_splits + blockIdx.x;
                float* dst = a.part_acc + idx * kTcD;
#pragma unroll 1
                for (int c0 = half * (kTcD / 2); c0 < (half + 1) * (kTcD / 2); c0 += 32) {
                    uint32_t rr[32];
                    tc::tmem_ld_32x32(tmem_o + lane_base + c0, rr);
                    tc::tmem_ld_wait();
                    if (mine) {
#pragma unroll
                        for (int jj = 0; jj < 32; jj += 4)
                            *reinterpret_cast<uint4*>(dst + c0 + jj) = make_uint4(rr[jj], rr[jj + 1], rr[jj + 2], rr[jj + 3]);
                    }
                }
                if (mine && half == 0) {
                    const float l = l_run + s_l[1][row];
                    a.part_ml[idx * 2] = l > 0.f ? m_ref * 0.6931471805599453f : -3.0e38f;
                    a.part_ml[idx * 2 + 1] = l;
                }
            }
        } else {
        if (ok) {
            tc::fence_after_sync();
            const float l = l_run + s_l[half ^ 1][row];
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem) + row * kTcOutPitch;
#pragma unroll 1
            for (int c0 = half * (kTcD / 2); c0 < (half + 1) * (kTcD / 2); c0 += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_o + lane_base + c0, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        w[e] = f32x2_to_bf16x2_bits(__uint_as_float(r[j + 2 * e]) * inv, __uint_as_float(r[j + 2 * e + 1]) * inv);
                    *reinterpret_cast<uint4*>(stg + c0 + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        if (cta_stamp) a.prof[4 * 16 + 15] = clock64();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (cta_stamp) a.prof[5 * 16 + 15] = clock64();
        if (ok) {
            // 16-byte pieces, four per thread and pass so that the gate loads of a pass are in flight together
            const __nv_bfloat16* stg0 = reinterpret_cast<const __nv_bfloat16*>(smem);
            const int n_items = nq * (kTcD / 8);
            for (int i0 = (int)threadIdx.x; i0 < n_items; i0 += 8 * kTcRows) {
                uint4 g[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * 2 * kTcRows;
                    g[u] = make_uint4(0, 0, 0, 0);
                    if (a.gate != nullptr && i < n_items)
                        g[u] = __ldg(reinterpret_cast<const uint4*>(a.gate + (size_t)(row_start + r_begin + (i >> 5)) * a.ld_gate +
                                                                    (size_t)h * a.gate_head_stride + a.gate_offset + (i & 31) * 8));
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * 2 * kTcRows;
                    if (i >= n_items) break;
                    const int r = i >> 5, c = i & 31;
                    uint4 v = *reinterpret_cast<const uint4*>(stg0 + r * kTcOutPitch + c * 8);
                    if (a.gate != nullptr) {
                        const uint32_t vw[4] = {v.x, v.y, v.z, v.w}, gw[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 vv = bf16x2_bits_to_f32x2(vw[e]), gg = bf16x2_bits_to_f32x2(gw[e]);
                            o[e] = f32x2_to_bf16x2_bits(vv.x * sigmoid_fast(gg.x), vv.y * sigmoid_fast(gg.y));
                        }
                        v = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    *reinterpret_cast<uint4*>(a.out + ((size_t)(row_start + r_begin + r) * a.Hq + h) * kTcD + c * 8) = v;
                }
            }
        }
        }   // prefill epilogue
    }
    if (cta_stamp) a.prof[6 * 16 + 15] = clock64();
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_bad != 0) set_status(a.status, PS_DEV_BAD_INDEX);
        if (s_abort != 0) {
            set_status(a.status, PS_DEV_WAIT_TIMEOUT);
            // copies still in flight get a bounded chance to land before the shared memory goes back to the next CTA
            const long long bd = a.budget < 4000000ll ? a.budget : 4000000ll;
            if (q_issued > q_consumed) tc::mbar_wait(&q_full, 0, bd);
            for (int c = k_consumed; c < k_issued; ++c) tc::mbar_wait(&k_full[c & 1], (uint32_t)(c >> 1) & 1u, bd);
            for (int c = v_consumed; c < v_issued; ++c) tc::mbar_wait(&v_full[c & 1], (uint32_t)(c >> 1) & 1u, bd);
        }
    }
    __syncthreads();
    if (cta_stamp) a.prof[16 + 15] = clock64();
    if (warp == 12) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem, kTcTmemCols);
    }
}

// FP8 pools: the sequences' pages are widened once per layer and step into a bf16 scratch pool of the same page shape
// (values times their per-token scale), with its own block table (scratch page = running index) and sequence descriptors
// (slot = sequence index), and the tensor-core kernel runs on that.  The copy moves 3 bytes per cached element; the
// attention it feeds is an order of magnitude faster than the mma.sync kernel on FP8 pages.
struct AttnDeqArgs {
    const uint8_t* k_pool; const uint8_t* v_pool; const float* k_scale; const float* v_scale;
    const int* block_table; int max_blocks; int num_pages; int page_tokens; int Hkv;
    const int* seqs; int n_seqs; int min_rows;
    __nv_bfloat16* k_out; __nv_bfloat16* v_out; int out_pages;
    int* bt_out;                 // [n_seqs][max_blocks]
    int* seqs_out;               // [n_seqs][4]
    uint32_t* status;
};

// grid = (scratch pages, Hkv), block = 256
__global__ void __launch_bounds__(256) attn_kv_dequant_kernel(const AttnDeqArgs a) {
    const int p = blockIdx.x, kvh = blockIdx.y, pt = a.page_tokens;
    // which sequence and block this scratch page belongs to
    int base = 0, s = 0, blk = -1, kv_end = 0, slot = -1;
    for (; s < a.n_seqs; ++s) {
        const int* sd = a.seqs + 4 * s;
        const int n_rows = sd[1];
        if (sd[2] < 0 || n_rows <= a.min_rows) continue;
        const int end = sd[3] + n_rows, np = (end + pt - 1) / pt;
        if (p < base + np) { blk = p - base; kv_end = end; slot = sd[2]; break; }
        base += np;
    }
    if (p == 0 && kvh == 0) {
        for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x) {
            const int* sd = a.seqs + 4 * i;
            a.seqs_out[4 * i + 0] = sd[0]; a.seqs_out[4 * i + 1] = sd[1]; a.seqs_out[4 * i + 2] = sd[2] < 0 ? -1 : i; a.seqs_out[4 * i + 3] = sd[3];
        }
    }
    if (blk < 0) return;
    if (kvh == 0 && threadIdx.x == 0) a.bt_out[(size_t)s * a.max_blocks + blk] = p;
    const int page = a.block_table[(size_t)slot * a.max_blocks + blk];
    const bool ok = page >= 0 && page < a.num_pages;
    if (!ok && threadIdx.x == 0) set_status(a.status, PS_DEV_BAD_INDEX);
    const size_t src = ((size_t)(ok ? page : 0) * a.Hkv + kvh) * pt;          // token rows of the source page
    const size_t dst = ((size_t)p * a.Hkv + kvh) * pt;
    for (int i = threadIdx.x; i < pt * (kTcD / 16); i += blockDim.x) {
        const int tok = i / (kTcD / 16), c = i % (kTcD / 16);
        const bool live = ok && blk * pt + tok < kv_end;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const uint8_t* pool = which ? a.v_pool : a.k_pool;
            const float* sp = which ? a.v_scale : a.k_scale;
            __nv_bfloat16* out = which ? a.v_out : a.k_out;
            uint32_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (live) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(pool + (src + tok) * kTcD) + c);
                const float sc = sp[src + tok];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float lo = e4m3_to_f32((w[j >> 1] >> ((j & 1) * 16)) & 0xff) * sc;
                    const float hi = e4m3_to_f32((w[j >> 1] >> ((j & 1) * 16 + 8)) & 0xff) * sc;
                    o[j] = f32x2_to_bf16x2_bits(lo, hi);
                }
            }
            uint4* d = reinterpret_cast<uint4*>(out + (dst + tok) * kTcD + c * 16);
            d[0] = make_uint4(o[0], o[1], o[2], o[3]);
            d[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
}

typedef CUresult (*EncodeTiledFnA)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnA attn_encode_fn() {
    static EncodeTiledFnA fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFnA>(p);
    }
    return fn;
}

// bf16 row-major [rows, cols] (leading dimension in elements) with a (box_rows x 64) box and the 128-byte swizzle.
static int attn_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows) {
    EncodeTiledFnA enc = attn_encode_fn();
    if (enc == nullptr) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld_elems * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static long long* g_attn_tc_prof = nullptr;

// True when the tensor-core kernel can take the call (the caller falls back to the mma.sync kernel otherwise).
bool attn_prefill_tc_supported(int D, int page_tokens, int kv_fp8, const void* q, const void* k_pool, const void* v_pool,
                               const void* gate, int ld_gate, int gate_head_stride, int gate_offset, const void* deq_k) {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("PS_ATTN_PREFILL");                 // "legacy": always the mma.sync kernel
        enabled = (e != nullptr && e[0] == 'l') ? 0 : 1;
    }
    if (!enabled || D != kTcD || (page_tokens != 16 && page_tokens != 32 && page_tokens != 64) || (kv_fp8 && deq_k == nullptr)) return false;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) % 16) return false;
    if (gate != nullptr && (((uintptr_t)gate % 16) || (ld_gate % 8) || (gate_head_stride % 8) || (gate_offset % 8))) return false;
    return true;
}

int launch_attn_prefill_tc(const void* q, int q_rows, const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale,
                           int kv_fp8, const void* block_table, int max_blocks, int num_pages, int page_tokens, const void* seqs,
                           int n_seqs, int max_seq_rows, int min_rows, int Hq, int Hkv, float sm_scale, const void* gate, int ld_gate,
                           int gate_head_stride, int gate_offset, void* deq_k, void* deq_v, int deq_pages, void* deq_bt, void* deq_seqs,
                           void* out, void* status, cudaStream_t stream) {
    if (kv_fp8) {
        // widen the step's pages into the bf16 scratch pool, then attend over that
        if (deq_k == nullptr || deq_v == nullptr || deq_bt == nullptr || deq_seqs == nullptr || deq_pages <= 0) return (int)cudaErrorInvalidValue;
        AttnDeqArgs d;
        d.k_pool = (const uint8_t*)k_pool; d.v_pool = (const uint8_t*)v_pool; d.k_scale = (const float*)k_scale; d.v_scale = (const float*)v_scale;
        d.block_table = (const int*)block_table; d.max_blocks = max_blocks; d.num_pages = num_pages; d.page_tokens = page_tokens; d.Hkv = Hkv;
        d.seqs = (const int*)seqs; d.n_seqs = n_seqs; d.min_rows = min_rows; d.k_out = (__nv_bfloat16*)deq_k; d.v_out = (__nv_bfloat16*)deq_v;
        d.out_pages = deq_pages; d.bt_out = (int*)deq_bt; d.seqs_out = (int*)deq_seqs; d.status = (uint32_t*)status;
        attn_kv_dequant_kernel<<<dim3(deq_pages, Hkv), 256, 0, stream>>>(d);
        int e = PS_LAUNCH_CHECK();
        if (e) return e;
        k_pool = deq_k; v_pool = deq_v; block_table = deq_bt; seqs = deq_seqs; num_pages = deq_pages;
    }
    CUtensorMap mq, mk, mv;
    int err = attn_map_2d(&mq, q, (uint64_t)q_rows, (uint64_t)Hq * kTcD, (uint64_t)Hq * kTcD, kTcRows);
    if (err) return err;
    const uint64_t pool_rows = (uint64_t)num_pages * Hkv * page_tokens;
    if ((err = attn_map_2d(&mk, k_pool, pool_rows, kTcD, kTcD, (uint32_t)page_tokens))) return err;
    if ((err = attn_map_2d(&mv, v_pool, pool_rows, kTcD, kTcD, (uint32_t)page_tokens))) return err;
    AttnTcArgs a;
    a.block_table = (const int*)block_table; a.max_blocks = max_blocks; a.num_pages = num_pages; a.page_tokens = page_tokens; a.seqs = (const int*)seqs;
    a.Hq = Hq; a.Hkv = Hkv; a.scale_log2 = sm_scale * 1.4426950408889634f; a.min_rows = min_rows;
    a.gate = (const __nv_bfloat16*)gate; a.ld_gate = ld_gate; a.gate_head_stride = gate_head_stride; a.gate_offset = gate_offset;
    a.out = (__nv_bfloat16*)out; a.status = (uint32_t*)status; a.budget = g_ps_wait_budget_cycles; a.prof = g_attn_tc_prof;
    a.split_tokens = 0; a.max_splits = 0; a.dec_max_rows = 0; a.part_acc = nullptr; a.part_ml = nullptr;
    const size_t smem = (size_t)kTcSmem;
    static bool set = false;
    if (!set) {
        cudaFuncSetAttribute(attn_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        set = true;
    }
    const int tiles = (max_seq_rows + kTcRows - 1) / kTcRows;
    attn_tc_kernel<false><<<dim3(tiles, Hq, n_seqs), kTcThreads, smem, stream>>>(mq, mk, mv, a);
    return PS_LAUNCH_CHECK();
}

}  // namespace ps

// Decode / verify attention on the tensor cores (bf16 pools, head dim 256, pages of 16 / 32 / 64 tokens, at most 8 query
// heads per KV head): split-KV partials for every sequence of the step with at most `dec_max_rows` (<= 16) rows, in the
// layout of ps_paged_attention's merge pass (`part_acc` [rows, Hq, max_splits, D] fp32, `part_ml` [rows, Hq, max_splits, 2]);
// the caller runs ps_paged_attention_merge afterwards.  `split_tokens` is a multiple of 64, `q` is [q_rows, Hq, D] bf16.
// Reference: src/phaseshift/models/qwen35/kernels/optimized/attention/paged_decode.hip (split-KV decode); the grouped-query
// packing onto one MMA tile has no counterpart there.
PS_API int ps_attn_decode_tc(const void* q, int q_rows, const void* k_pool, const void* v_pool, const void* block_table,
                             int max_blocks, int page_tokens, int num_pages, const void* seqs, int n_seqs, int dec_max_rows,
                             int Hq, int Hkv, int D, float sm_scale, int split_tokens, int max_splits, int max_visible,
                             void* part_acc, void* part_ml, void* status, cudaStream_t stream) {
    using namespace ps;
    if (D != kTcD || (page_tokens != 16 && page_tokens != 32 && page_tokens != 64) || Hkv <= 0 || (Hq % Hkv) || Hq / Hkv > 8 ||
        dec_max_rows < 1 || dec_max_rows > 16 || split_tokens < kTcTok || (split_tokens % kTcTok) || n_seqs <= 0 ||
        (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)part_acc) % 16))
        return (int)cudaErrorInvalidValue;
    int n_splits = (max_visible + split_tokens - 1) / split_tokens;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > max_splits) return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mk, mv;
    int err = attn_map_2d(&mq, q, (uint64_t)q_rows * Hq, kTcD, kTcD, 8);                 // the [rows * Hq, D] view, 8-row boxes
    if (err) return err;
    const uint64_t pool_rows = (uint64_t)num_pages * Hkv * page_tokens;
    if ((err = attn_map_2d(&mk, k_pool, pool_rows, kTcD, kTcD, (uint32_t)page_tokens))) return err;
    if ((err = attn_map_2d(&mv, v_pool, pool_rows, kTcD, kTcD, (uint32_t)page_tokens))) return err;
    AttnTcArgs a;
    a.block_table = (const int*)block_table; a.max_blocks = max_blocks; a.num_pages = num_pages; a.page_tokens = page_tokens; a.seqs = (const int*)seqs;
    a.Hq = Hq; a.Hkv = Hkv; a.scale_log2 = sm_scale * 1.4426950408889634f; a.min_rows = 0;
    a.gate = nullptr; a.ld_gate = 0; a.gate_head_stride = 0; a.gate_offset = 0; a.out = nullptr;
    a.status = (uint32_t*)status; a.budget = g_ps_wait_budget_cycles; a.prof = nullptr;
    a.split_tokens = split_tokens; a.max_splits = max_splits; a.dec_max_rows = dec_max_rows;
    a.part_acc = (float*)part_acc; a.part_ml = (float*)part_ml;
    const size_t smem = (size_t)kTcSmem;
    static bool set = false;
    if (!set) {
        cudaFuncSetAttribute(attn_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        set = true;
    }
    attn_tc_kernel<true><<<dim3(n_splits, Hkv, n_seqs), kTcThreads, smem, stream>>>(mq, mk, mv, a);
    return PS_LAUNCH_CHECK();
}

// Timing aid: a device buffer of 32 x 16 int64 that CTA (0, 0, 0) of later launches fills with cycle stamps of its softmax
// thread 0 (slots 0-7: tile start, scores ready, scores loaded, row maximum exchanged, probabilities computed, stored,
// proxy fence done, arrived) and of the issuing threads (slots 8-10: score issuer at its tile's start, operands ready,
// issued; 11-12: output issuer with probabilities ready, issued; slot 15 of tiles 0 and 1: start and end of the CTA).  nullptr switches it off.
PS_API void ps_attn_prefill_tc_set_prof(void* buf) { ps::g_attn_tc_prof = (long long*)buf; }
