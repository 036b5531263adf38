// Block-scaled tensor-core projection: out[M, N] = epilogue( act[M, K] . W[N, K]^T ) with the quantised
// codes themselves as tensor-core operands (`tcgen05.mma.kind::mxf4nvf4` for NVFP4 weights,
// `kind::mxf8f6f4.block_scale` for MXFP8 weights).  One kernel serves decode (1 row), speculative
// verification (a few rows), batched decode and prefill (thousands of rows).
//
// Orientation.  The WEIGHT rows are always the M side of the instruction (tiles of 128 output
// features), the batch rows the N side (NB = 16 / 32 resident, 128 / 256 streamed).  So the accumulator
// in tensor memory has one output feature per lane and one batch row per column, and every byte a
// pipeline stage brings in for small batches is weight data: the projection is a stream over W.
//
// Operands.  Weight codes stay in their canonical row-major form ([N, K/2] nibbles or [N, K] bytes);
// a 2-D TMA tile load (128 rows x 128 bytes, 128-byte swizzle, no multicast) turns them into the
// shared-memory operand layout.  Block scales are stored once at load in 512-byte "atoms" (see
// ps_tcgen05.cuh) so that a stage's scales are one contiguous bulk copy followed by `tcgen05.cp`
// into tensor memory.  Activations are quantised to the same block format as the weights
// (NVFP4 weights: E2M1 + UE4M3 per 16 with a fixed per-projection scale; MXFP8 weights: E4M3 + UE8M0
// per 32):
//   * resident path (M <= 32): the kernel's own prologue reads the bf16 rows, quantises the K-panels
//     this CTA needs and writes them, already swizzled, into shared memory where they stay for the
//     CTA's lifetime; their block scales go to tensor memory once (`tcgen05.st`), so a stage costs
//     only the weight-scale copies and four MMAs;
//   * streamed path: `ps_act_quant` has written codes + scale atoms to global memory and they travel
//     through the stage ring next to the weights.
// A fused RMSNorm(1 + w) is applied in two commuting halves: the element-wise factor (1 + w) before
// quantisation, the per-row factor 1/rms in the epilogue (a row scale commutes with the product).
// The row sums of squares come from the producing kernel's epilogue when it left per-tile partial
// sums (`ssq_in`), so the prologue is a single round trip of loads; otherwise the CTA sweeps the rows
// itself.  A residual epilogue can in turn leave the partial sums of what it stores (`ssq_out`).
//
// Work split (stream-K).  Work units are (tile, K-panel) pairs in tile-major order, cut into equal
// contiguous ranges, one per CTA (one CTA per SM), so every SM streams the same number of bytes for
// any N and K.  A tile cut over several CTAs is finished without anybody waiting: each contributor
// stores its fp32 partial in a workspace slot of its own and bumps the tile's arrival counter; the
// contributor that arrives last adds all partials in CTA order (the same sum whoever does it) and
// runs the epilogue.  The split is a function of (N, K, grid) only, never of
// M, and a column of the accumulator depends on its own batch row only, so row r of an M-row launch is
// bit-identical to the same row in a 1-row launch (the property speculative verification needs; the
// reference gets it from its ExactRows kernels, src/phaseshift/models/qwen35/kernels/optimized/
// linear/bf16.hip:429-512).
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and tensor-memory owner, warps 2..5 = epilogue
// (`tcgen05.ld`, fix-up, residual / SwiGLU / dtype, optional tensor-parallel combine over peer memory).
// Two accumulators (NB <= 128) let the epilogue of one segment overlap the MMAs of the next.  Every
// wait (mbarrier, stream-K flag, peer flag) is bounded by the launch's cycle budget; on expiry the CTA
// raises an abort flag, reports PS_DEV_WAIT_TIMEOUT, waits (bounded) for copies and MMAs in flight,
// frees its tensor memory and returns.
//
// Reference counterparts: the PSQ4 / PSQ8 W4A8 / W8A8 families (src/phaseshift/models/qwen35/kernels/
// optimized/linear/psq4.hip:221-349,505-667, linear/psq8.hip:161-518) and the activation quantiser
// (optimized/activation_quantize.hip:65-317).
#include <cuda_fp4.h>

#include "gemv_core.cuh"
#include "ps_tcgen05.cuh"

namespace ps {

constexpr int kBsThreads = 192;
constexpr int kBsTileN = 128;                       // weight rows per tile (the instruction's M)
constexpr int kBsATile = kBsTileN * 128;            // bytes of one weight stage tile
constexpr int kBsMaxStages = 12;
constexpr int kBsMaxTiles = 1 << 17;                // arrival counters a launch may use
constexpr int kBsSmemBudget = 222 * 1024;      // dynamic part; ~3 KB of static shared memory come on top (227 KB limit)

template <int FMT> struct BsT;
template <> struct BsT<W_NVFP4> { static constexpr int kPanelK = 256, kApp = 4, kBlockK = 16, kBpp = 16; };
template <> struct BsT<W_MXFP8> { static constexpr int kPanelK = 128, kApp = 1, kBlockK = 32, kBpp = 4; };

// Reduce-scatter by push (tensor-parallel row-parallel projections with many rows): rows are dealt to the ranks in
// contiguous blocks of `rpr`; the epilogue stores each bf16 row piece of this rank's partial product straight into the
// owner's receive buffer over NVLink (plain 16-byte peer stores, overlapping the main loop of the tiles still to come).
// The owner adds the `size` partials, the residual, and hands the rows to every rank (ps_tp_reduce_gather, allreduce.cu).
struct TpScatter {
    int size, rank, rpr, ld;              // size <= 1: disabled; ld = elements per row of the receive buffers
    __nv_bfloat16* recv[kTpMaxRanks];     // rank r's receive buffer: [size (source)][rpr][ld] bf16
};

struct BsArgs {
    int M, N, K;
    int P, tiles_n, tiles_m, total_units;
    const uint8_t* sfw;            // weight scale atoms [tiles_n][P * kApp][512]
    float out_scale;               // weight tensor scale x activation scale
    // resident activations (quantised in the prologue)
    const __nv_bfloat16* x; int ldx;
    const __nv_bfloat16* norm_w; float eps;
    float act_c1, act_gs;          // 1 / (6 gs), gs  (NVFP4 activations)
    __nv_bfloat16* xn_out;
    int res_slots, res_full;
    const float* ssq_in; int ssq_n, ssq_in_ld;      // per-row partial sums of squares of x left by its producer
    float* ssq_out; int ssq_out_ld;                 // residual epilogue: partial sums of squares of the stored rows
    const float* row_scale;                         // streamed path: per-row factor (1/rms) applied in the epilogue
    // streamed activations (quantised by ps_act_quant)
    const uint8_t* sfx;            // activation scale atoms [m blocks of 128][P * kApp][512]
    int epilogue;
    const __nv_bfloat16* residual; int ld_res;
    void* out; int ldo; int out_f32;
    float* ws; uint32_t* flags;    // stream-K partials [grid][2][NB][128] and per-tile arrival counters (zero between launches)
    uint32_t* status; long long budget;
    int stages;
    // L2 prefetch of the projection that runs next (its first ring fill per CTA); next_total == 0: none
    const uint8_t* next_sfw; int next_P, next_tiles_m, next_total, next_grid, next_stages, next_sf_bytes;
    long long* prof;               // optional [16] cycle stamps of CTA 0 (ps_gemm_bs_profile); null in normal use
    int dbg;                       // timing experiments only (PS_BS_DBG): 1 skip weight-scale copies, 2 skip activation-scale
                                   // copies, 4 skip MMAs, 8 skip the activation prologue; results are then meaningless
    TpCombine tp;
    TpScatter rs;                  // streamed path, tensor parallel: bf16 tiles go to the rank that owns their rows
};

// CTA that owns unit x under cta_range(total, grid, c, ...).
__host__ __device__ inline int unit_owner(int total, int grid, int x) {
    const int base = total / grid, rem = total % grid;
    const int boundary = rem * (base + 1);
    return x < boundary ? x / (base + 1) : rem + (x - boundary) / base;
}

// Walks a CTA's unit range as groups of up to G consecutive K-panels of one tile: one pipeline stage each.  Producer and
// consumers walk the same sequence (a segment of BsSegIter splits into the same groups).
struct BsGroupIter {
    int u, u_end, P, G;
    __device__ __forceinline__ bool next(int& t, int& p, int& gn) {
        if (u >= u_end) return false;
        t = u / P; p = u - t * P;
        gn = min(G, min(P - p, u_end - u));
        u += gn;
        return true;
    }
};

// Walks a CTA's unit range as segments (tile, [p0, p1)).
struct BsSegIter {
    int u, u_end, P;
    __device__ __forceinline__ bool next(int& t, int& p0, int& p1) {
        if (u >= u_end) return false;
        t = u / P; p0 = u - t * P;
        p1 = min(P, p0 + (u_end - u));
        u += p1 - p0;
        return true;
    }
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// ---- activation block quantisers (shared by the resident prologue and ps_act_quant)
// 16 values -> 8 bytes of E2M1 (byte j = q[2j] | q[2j+1] << 4) + one UE4M3 scale byte.
__device__ __forceinline__ void quant_block_nvfp4(const float (&v)[16], float c1, float gs, uint2& codes, uint8_t& sf) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    sf = f32_to_e4m3(__fmul_rn(amax, c1));
    const float sf_f = e4m3_to_f32(sf);
    const float inv = sf_f > 0.f ? __fdiv_rn(1.f, __fmul_rn(sf_f, gs)) : 0.f;
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t acc = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 pr = make_float2(__fmul_rn(v[h * 8 + 2 * j], inv), __fmul_rn(v[h * 8 + 2 * j + 1], inv));
            acc |= (uint32_t)__nv_cvt_float2_to_fp4x2(pr, __NV_E2M1, cudaRoundNearest) << (8 * j);
        }
        w[h] = acc;
    }
    codes = make_uint2(w[0], w[1]);
}
// 32 values -> 32 E4M3 bytes + one UE8M0 exponent byte (largest power of two with amax / 2^e <= 448).
__device__ __forceinline__ void quant_block_mxfp8(const float (&v)[32], uint4 (&codes)[2], uint8_t& sf) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    int e = 0;
    if (amax >= 1e-30f) {
        const uint32_t bits = __float_as_uint(amax);
        const int ea = (int)((bits >> 23) & 0xffu) - 127;
        const float mant = __uint_as_float((bits & 0x007fffffu) | 0x3f800000u);
        e = ea - 8 + (mant > 1.75f ? 1 : 0);
        e = max(-126, min(126, e));
    }
    sf = (uint8_t)(e + 127);
    const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint32_t acc = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b)
            acc |= (uint32_t)__nv_cvt_float_to_fp8(amax >= 1e-30f ? __fmul_rn(v[j * 4 + b], inv) : 0.f, __NV_SATFINITE, __NV_E4M3) << (8 * b);
        w[j] = acc;
    }
    codes[0] = make_uint4(w[0], w[1], w[2], w[3]);
    codes[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Load `n` (16 or 32) consecutive bf16 activations of a row, apply the fused RMSNorm when asked:
// v = bf16(x * inv_rms * (1 + w)), rounded like a stand-alone norm kernel would store it.
template <int NV>
__device__ __forceinline__ void load_act_block(const __nv_bfloat16* xr, const __nv_bfloat16* norm_w, int k0, int K,
                                               float inv_rms, float (&v)[NV]) {
#pragma unroll
    for (int q = 0; q < NV / 8; ++q) {
        const int k = k0 + q * 8;
        if (k < K) {      // K is a multiple of 8: a vector is entirely inside or outside
            const uint4 xv = *reinterpret_cast<const uint4*>(xr + k);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
            if (norm_w != nullptr) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(norm_w + k));
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 a = bf16x2_bits_to_f32x2(xw[e]), w = bf16x2_bits_to_f32x2(ww[e]);
                    v[q * 8 + 2 * e] = bf16_to_f32(f32_to_bf16(a.x * inv_rms * (1.f + w.x)));
                    v[q * 8 + 2 * e + 1] = bf16_to_f32(f32_to_bf16(a.y * inv_rms * (1.f + w.y)));
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 a = bf16x2_bits_to_f32x2(xw[e]);
                    v[q * 8 + 2 * e] = a.x; v[q * 8 + 2 * e + 1] = a.y;
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[q * 8 + e] = 0.f;
        }
    }
}

// Byte offset of scale factor (row r, atom-local K-block j) inside a 512-byte atom.
__host__ __device__ __forceinline__ int sf_atom_off(int r, int j) { return (r & 31) * 16 + ((r >> 5) & 3) * 4 + j; }

// Threads per CTA: warp 0 producer, warp 1 MMA issuer, warps 2..5 epilogue, warp 6 scale-copy issuer; the resident variant
// adds five more warps that only help in the activation prologue (one (slot, block) pair per thread instead of two in a row).
// Warp 6 issues the scale-factor copies (tcgen05.cp) one stage ahead of the MMA warp: the two instruction streams of a
// stage (copies: ~55 cycles each, MMAs: ~86 each at N = 16) run in parallel instead of back to back in one thread.
template <bool RES> constexpr int bs_threads() { return RES ? 384 : kBsThreads + 32; }
template <bool RES> constexpr int bs_group() { return RES ? 2 : 1; }      // K-panels per pipeline stage

template <int FMT, int NB, bool RES>
__global__ void __launch_bounds__(bs_threads<RES>(), 1)
gemm_bs_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_next, const BsArgs g) {
    using T = BsT<FMT>;
    constexpr int kThreads = bs_threads<RES>(), kWarps = kThreads / 32;
    constexpr int APP = T::kApp;
    constexpr int NBLK = NB > 128 ? 2 : 1;
    constexpr int kBTile = NB * 128;
    constexpr int kSfaBytes = APP * 512, kSfbBytes = NBLK * APP * 512;
    // Resident path: a pipeline stage holds G = 2 weight panels, so the MMA thread's per-stage costs (two barrier waits, the
    // commit, loop control: ~600 of ~920 cycles per 16 KB panel, measured) are paid once per 32 KB.
    constexpr int G = bs_group<RES>();
    constexpr int kStageRaw = RES ? G * (kBsATile + kSfaBytes) : (kBsATile + kBTile + kSfaBytes + kSfbBytes);
    constexpr int kStage = (kStageRaw + 1023) / 1024 * 1024;
    constexpr int kOffB = kBsATile;
    constexpr int kOffSfa = RES ? G * kBsATile : kBsATile + kBTile;
    constexpr int kOffSfb = kOffSfa + kSfaBytes;
    constexpr uint32_t kPanelTx = RES ? (kBsATile + kSfaBytes) : (kBsATile + kBTile + kSfaBytes + kSfbBytes);   // bytes per panel of a stage
    constexpr int kResSfWords = APP * 32;           // resident path: 32-bit scale words per panel slot (4 K-blocks each)
    constexpr int ACC_BUFS = NB <= 128 ? 2 : 1;
    constexpr int ACC_STRIDE = NB < 32 ? 32 : NB;
    constexpr uint32_t SF_COL0 = ACC_BUFS * ACC_STRIDE;
    constexpr uint32_t SFA_COLS = 4 * APP, SFB_COLS = RES ? 0 : 4 * APP * NBLK, SF_BUF_COLS = G * SFA_COLS + SFB_COLS;
    // resident activation scales: one 4-column granule per (slot, K-block group), like a tcgen05.cp would fill;
    // only the first column of a granule is written and read (batch rows < 32), but the MMA's scale address
    // stays 4-column aligned
    // Streamed path: warp 6 issues the scale-factor copies ahead of the MMA warp (12 copies per stage would otherwise sit in
    // front of 4 MMAs in one instruction stream: +19 % at 2048 rows).  Resident path: 4 copies per stage, the hand-over between
    // two threads costs more than it saves (measured), so the MMA thread issues them itself.
    constexpr bool kSplitSf = !RES;
    constexpr int kSfBufs = kSplitSf ? 4 : 2;        // scale-factor column sets in flight
    constexpr uint32_t SFB_RES_COL0 = SF_COL0 + kSfBufs * SF_BUF_COLS;
    static_assert(SF_COL0 + kSfBufs * SF_BUF_COLS <= 512, "tensor memory budget");
    constexpr int CH = NB == 16 ? 16 : 32;          // accumulator columns read per tcgen05.ld

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sBres = smem + (size_t)g.stages * kStage;                          // resident activation codes
    __nv_bfloat16* sEpi = reinterpret_cast<__nv_bfloat16*>(sBres);                    // streamed path: 128 x 128 bf16 output staging
    uint32_t* sSfRes = reinterpret_cast<uint32_t*>(sBres + (size_t)g.res_slots * kBTile);   // [slot][APP][32 rows] scale words
    __shared__ __align__(8) uint64_t full_bar[kBsMaxStages], empty_bar[kBsMaxStages], acc_full[2], acc_empty[2], drain_bar;
    __shared__ __align__(8) uint64_t sf_ready[4], sf_free[4];      // scale-factor columns of a stage parity: copied / consumed
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int s_abort;
    __shared__ int s_issued, s_consumed;
    __shared__ float s_inv_rms[32], s_red[32 * kWarps], s_ssq[4 * 32];

    cudaTriggerProgrammaticLaunchCompletion();
    const bool prof = g.prof != nullptr && blockIdx.x == 0;
    if (prof && threadIdx.x == 0) g.prof[0] = clock64();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int P = g.P, stages = g.stages;
    int u0, u1;
    cta_range(g.total_units, gridDim.x, blockIdx.x, u0, u1);

    // ---- set-up: the barriers are initialised by two threads in parallel, then thread 0 at once fills the ring
    // with weights (they do not depend on the stream predecessor) while warps 1..5 go on to the prologue
    // weights (and their scale atoms) of one group into stage slot `slot`
    auto issue_weights = [&](int slot, int t, int p, int gn) {
        const int tn = t / g.tiles_m;
        unsigned char* st = smem + (size_t)slot * kStage;
        tc::mbar_expect_tx(&full_bar[slot], (uint32_t)gn * kPanelTx);
        for (int j = 0; j < gn; ++j) {
            tc::tma_load_2d(st + j * kBsATile, &map_w, (p + j) * 128, tn * kBsTileN, &full_bar[slot]);
            tc::bulk_load(st + kOffSfa + j * kSfaBytes, g.sfw + ((size_t)tn * P + p + j) * kSfaBytes, kSfaBytes, &full_bar[slot]);
        }
    };
    BsGroupIter GI{u0, u1, P, G};               // thread 0's walk: ring fill here, the rest in the producer role
    int pre = 0;                                // groups issued before the dependency sync (thread 0 only)
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) tc::mbar_init(&full_bar[s], 1);
        tc::fence_barrier_init();
        s_abort = 0; s_issued = 0; s_consumed = 0;
        int t, p, gn;
        while (pre < stages && GI.next(t, p, gn)) { issue_weights(pre, t, p, gn); ++pre; }
        if (!RES) tc::tma_prefetch_desc(&map_x);
    } else if (threadIdx.x == 64) {
        for (int s = 0; s < stages; ++s) tc::mbar_init(&empty_bar[s], 1);
        for (int b = 0; b < 2; ++b) { tc::mbar_init(&acc_full[b], 1); tc::mbar_init(&acc_empty[b], 4); }
        tc::mbar_init(&drain_bar, 1);
        for (int b = 0; b < 4; ++b) { tc::mbar_init(&sf_ready[b], 1); tc::mbar_init(&sf_free[b], 1); }
        tc::fence_barrier_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(&tmem_base_slot, 512);
        tc::tmem_relinquish();
    }
    // ---- resident prologue, part 1 (before the stream predecessor is done): work split and the norm weights of this
    // thread's first blocks -- constants, usually a cold read from DRAM, so they are fetched while waiting
    constexpr int NVEC = T::kBlockK / 8;                  // 16-byte vectors per block
    constexpr int RB = 4;                                 // rows whose loads are issued together
    constexpr int kPreW = 2;                              // pairs whose norm weights are fetched ahead
    constexpr int kQThreads = kThreads - 32;              // every warp but warp 0, which is filling the ring
    const int qtid = (int)threadIdx.x - 32;
    const bool norm = RES && g.norm_w != nullptr;
    const int pairs = g.res_slots * T::kBpp;
    const int my_pairs = (RES && qtid >= 0 && qtid < pairs) ? (pairs - qtid + kQThreads - 1) / kQThreads : 0;
    uint4 wpre[kPreW][NVEC];
#pragma unroll
    for (int pl = 0; pl < kPreW; ++pl) {
        const int pi = qtid + kQThreads * pl;
        const int s = pi / T::kBpp, blk = pi - s * T::kBpp;
        const int p = g.res_full ? s : (u0 + s) % P;
        const int k0 = p * T::kPanelK + blk * T::kBlockK;
#pragma unroll
        for (int v4 = 0; v4 < NVEC; ++v4)
            wpre[pl][v4] = (norm && pl < my_pairs && k0 + v4 * 8 < g.K) ? __ldg(reinterpret_cast<const uint4*>(g.norm_w + k0 + v4 * 8))
                                                                         : make_uint4(0, 0, 0, 0);
    }
    if (prof && threadIdx.x == 32) g.prof[1] = clock64();
    cudaGridDependencySynchronize();
    if (prof && threadIdx.x == 32) g.prof[2] = clock64();

    if (RES && !(g.dbg & 8)) {
        // ---- prologue: block quantisation of x (1 + w) for the K-panels this CTA needs, row statistics
        // Only live rows are quantised: an accumulator column depends on its own batch row alone, so whatever the
        // rows >= M of the operand hold never reaches a stored value.  A thread takes (panel slot, block) pairs and
        // walks the rows RB at a time, all loads of a row group issued before the first conversion.
        // row statistics from the producer's partial sums: one thread per row, issued before the quantisation loads
        float ssq_acc = 0.f;
        if (norm && g.ssq_in != nullptr && qtid >= 0 && qtid < g.M) {
            // up to 64 partials per row, fetched as 16 independent vector loads (one round trip), added in order
            const float4* sp = reinterpret_cast<const float4*>(g.ssq_in + (size_t)qtid * g.ssq_in_ld);
            float4 pv[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) pv[i] = 4 * i < g.ssq_n ? __ldcg(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float e[4] = {pv[i].x, pv[i].y, pv[i].z, pv[i].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) if (4 * i + j < g.ssq_n) ssq_acc += e[j];
            }
        }
        for (int pl = 0; pl < my_pairs; ++pl) {
            const int pi = qtid + kQThreads * pl;
            const int s = pi / T::kBpp, blk = pi - s * T::kBpp;
            const int p = g.res_full ? s : (u0 + s) % P;
            const int k0 = p * T::kPanelK + blk * T::kBlockK;
            uint4 wv[NVEC];
            if (pl < kPreW) {
#pragma unroll
                for (int v4 = 0; v4 < NVEC; ++v4) wv[v4] = pl == 0 ? wpre[0][v4] : wpre[1][v4];
            } else {
#pragma unroll
                for (int v4 = 0; v4 < NVEC; ++v4)
                    wv[v4] = (norm && k0 + v4 * 8 < g.K) ? __ldg(reinterpret_cast<const uint4*>(g.norm_w + k0 + v4 * 8)) : make_uint4(0, 0, 0, 0);
            }
            unsigned char* cslot = sBres + (size_t)s * kBTile;
            uint8_t* sfw8 = reinterpret_cast<uint8_t*>(sSfRes + (size_t)s * kResSfWords);
            for (int r0 = 0; r0 < g.M; r0 += RB) {
                uint4 xv[RB][NVEC];
#pragma unroll
                for (int rr = 0; rr < RB; ++rr)
#pragma unroll
                    for (int v4 = 0; v4 < NVEC; ++v4)
                        xv[rr][v4] = (r0 + rr < g.M && k0 + v4 * 8 < g.K)
                                         ? *reinterpret_cast<const uint4*>(g.x + (size_t)(r0 + rr) * g.ldx + k0 + v4 * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int rr = 0; rr < RB; ++rr) {
                    const int r = r0 + rr;
                    if (r >= g.M) break;
                    float v[T::kBlockK];
#pragma unroll
                    for (int v4 = 0; v4 < NVEC; ++v4) {
                        const uint32_t xw[4] = {xv[rr][v4].x, xv[rr][v4].y, xv[rr][v4].z, xv[rr][v4].w};
                        const uint32_t ww[4] = {wv[v4].x, wv[v4].y, wv[v4].z, wv[v4].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 a2 = bf16x2_bits_to_f32x2(xw[e]), w2 = bf16x2_bits_to_f32x2(ww[e]);
                            v[v4 * 8 + 2 * e] = __fmul_rn(a2.x, 1.f + w2.x);        // w reads 0 without a norm
                            v[v4 * 8 + 2 * e + 1] = __fmul_rn(a2.y, 1.f + w2.y);
                        }
                    }
                    unsigned char* crow = cslot + (r >> 3) * 1024 + (r & 7) * 128;
                    if constexpr (FMT == W_NVFP4) {
                        uint2 codes; uint8_t sf;
                        quant_block_nvfp4(v, g.act_c1, g.act_gs, codes, sf);
                        *reinterpret_cast<uint2*>(crow + (((blk >> 1) ^ (r & 7)) << 4) + (blk & 1) * 8) = codes;
                        sfw8[((blk >> 2) * 32 + r) * 4 + (blk & 3)] = sf;
                    } else {
                        uint4 codes[2]; uint8_t sf;
                        quant_block_mxfp8(v, codes, sf);
                        *reinterpret_cast<uint4*>(crow + (((2 * blk) ^ (r & 7)) << 4)) = codes[0];
                        *reinterpret_cast<uint4*>(crow + (((2 * blk + 1) ^ (r & 7)) << 4)) = codes[1];
                        sfw8[r * 4 + blk] = sf;
                    }
                }
            }
        }
        if (prof && threadIdx.x == 32) g.prof[3] = clock64();
        if (norm) {
            if (g.ssq_in != nullptr) {
                if (qtid >= 0 && qtid < g.M) {
                    s_inv_rms[qtid] = rsqrtf(ssq_acc / (float)g.K + g.eps);
                    // statistics handed over by another kernel: a sum of squares is never negative, so a negative value means
                    // that its producer did not write it (the quantiser below would turn the damage into finite codes).
                    // Non-finite sums are left alone: padding rows of a bucket legitimately carry garbage through the layers.
                    if (ssq_acc < 0.f && blockIdx.x == 0) set_status(g.status, PS_DEV_NONFINITE);
                }
            } else {
                // No partial sums from a producer: sweep the rows here.  Thread t always adds elements t, t + kThreads, ...
                // of a row and the warp sums are added in warp order, so a row's statistics do not depend on how
                // many rows the launch has; four rows are swept together only to keep more loads in flight.
                const int kv = g.K >> 3;
                for (int m0 = 0; m0 < g.M; m0 += 4) {
                    float ss[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int i = threadIdx.x; i < kv; i += kThreads) {
#pragma unroll
                        for (int rr = 0; rr < 4; ++rr) {
                            if (m0 + rr < g.M) {
                                const uint4 x4 = *(reinterpret_cast<const uint4*>(g.x + (size_t)(m0 + rr) * g.ldx) + i);
                                const uint32_t xw[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                                for (int e = 0; e < 4; ++e) { const float2 a2 = bf16x2_bits_to_f32x2(xw[e]); ss[rr] += a2.x * a2.x + a2.y * a2.y; }
                            }
                        }
                    }
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) {
                        const float sv = warp_sum(ss[rr]);
                        if (lane == 0 && m0 + rr < g.M) s_red[(m0 + rr) * kWarps + warp] = sv;
                    }
                }
                __syncthreads();
                if ((int)threadIdx.x < g.M) {
                    float sv = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < kWarps; ++w2) sv += s_red[threadIdx.x * kWarps + w2];
                    s_inv_rms[threadIdx.x] = rsqrtf(sv / (float)g.K + g.eps);
                }
            }
        } else if ((int)threadIdx.x < 32) {
            s_inv_rms[threadIdx.x] = 1.f;
        }
        if (prof && threadIdx.x == 32) g.prof[4] = clock64();
    }
    // first CTA-wide barrier: barrier objects, the tensor-memory base and (resident path) the quantised panels
    if (RES) tc::fence_proxy_async_smem();  // generic-proxy writes of the codes -> visible to tcgen05.mma
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    if constexpr (RES) {
        if (warp >= 2 && warp < 6) {
            // activation block scales -> tensor memory, once: lane = batch row, APP columns per panel slot, the same
            // words in each of the four 32-lane sub-partitions (warp w writes its own)
            const uint32_t tcol = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SFB_RES_COL0;
            for (int s = 0; s < g.res_slots; ++s) {
                const uint32_t* wsrc = sSfRes + (size_t)s * kResSfWords + lane;
                if constexpr (APP == 4) tc::tmem_st_32x16_sparse4(tcol + 16 * (uint32_t)s, wsrc[0], wsrc[32], wsrc[64], wsrc[96]);
                else tc::tmem_st_32x1(tcol + 4 * (uint32_t)s, wsrc[0]);
            }
            tc::tmem_st_wait();
        }
        if (g.xn_out != nullptr && blockIdx.x == 0 && norm) {
            for (int i = threadIdx.x; i < g.M * (g.K >> 3); i += kThreads) {
                const int m = i / (g.K >> 3), k = (i % (g.K >> 3)) << 3;
                float v[8];
                load_act_block<8>(g.x + (size_t)m * g.ldx, g.norm_w, k, g.K, s_inv_rms[m], v);
                *reinterpret_cast<uint4*>(g.xn_out + (size_t)m * g.K + k) =
                    make_uint4(f32x2_to_bf16x2_bits(v[0], v[1]), f32x2_to_bf16x2_bits(v[2], v[3]),
                               f32x2_to_bf16x2_bits(v[4], v[5]), f32x2_to_bf16x2_bits(v[6], v[7]));
            }
        }
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();
    }
    if (prof && threadIdx.x == 32) g.prof[5] = clock64();

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int issued = pre;
            // activation half of a (single-panel) stage of the streamed path
            auto issue_acts = [&](int slot, int t, int p) {
                const int tm = t % g.tiles_m;
                unsigned char* st = smem + (size_t)slot * kStage;
                tc::tma_load_2d(st + kOffB, &map_x, p * 128, tm * NB, &full_bar[slot]);
#pragma unroll
                for (int j = 0; j < NBLK; ++j)
                    tc::bulk_load(st + kOffSfb + j * kSfaBytes, g.sfx + ((size_t)(tm * NBLK + j) * P + p) * kSfaBytes, kSfaBytes, &full_bar[slot]);
            };
            if constexpr (!RES) {
                for (int i = 0; i < pre; ++i) {     // activation halves of the stages filled before the dependency sync
                    const int u = u0 + i, t = u / P;
                    issue_acts(i, t, u - t * P);
                }
            }
            long long prof_pwait = 0;
            int t, p, gn;
            for (int it = pre; GI.next(t, p, gn); ++it) {
                const int s = it % stages;
                const long long tp0 = prof ? clock64() : 0;
                if (!tc::mbar_wait_abortable(&empty_bar[s], (uint32_t)((it / stages) & 1) ^ 1u, g.budget, &s_abort)) break;
                if (prof) prof_pwait += clock64() - tp0;
                issue_weights(s, t, p, gn);
                if constexpr (!RES) issue_acts(s, t, p);
                issued = it + 1;
            }
            s_issued = issued;
            if (prof) g.prof[14] = prof_pwait;
            if (g.next_total > 0 && (int)blockIdx.x < g.next_grid) {
                // everything this CTA needs is on its way: warm L2 with what the same CTA index reads first in the
                // projection that follows, so that kernel's ring fill does not start from DRAM
                int n0, n1;
                cta_range(g.next_total, g.next_grid, blockIdx.x, n0, n1);
                const int cnt = min(n1 - n0, g.next_stages * G);
                for (int i = 0; i < cnt; ++i) {
                    const int u = n0 + i, t = u / g.next_P, p = u - t * g.next_P, tn = t / g.next_tiles_m;
                    tc::tma_prefetch_l2_2d(&map_next, p * 128, tn * kBsTileN);
                    tc::bulk_prefetch_l2(g.next_sfw + ((size_t)tn * g.next_P + p) * g.next_sf_bytes, (uint32_t)g.next_sf_bytes);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            int it = 0, pi = 0, seg = 0, t, p0, p1, s = 0;      // it: stages consumed, pi: panels consumed
            uint32_t full_phase = 0;
            BsSegIter S{u0, u1, P};
            bool ok = true;
            long long prof_wait = 0, prof_sf = 0, prof_mma = 0, prof_commit = 0;
            // descriptor low words (address >> 4) of stage 0; a stage adds kStage >> 4, a K-block 2 (32 bytes)
            const uint32_t a_lo0 = ((tc::smem_u32(smem) >> 4) & 0x3FFFu) | tc::kDescSw128LoFlags;
            const uint32_t sfa_lo0 = (tc::smem_u32(smem + kOffSfa) >> 4) & 0x3FFFu;
            const uint32_t bres_lo0 = ((tc::smem_u32(sBres) >> 4) & 0x3FFFu) | tc::kDescSw128LoFlags;
            while (ok && S.next(t, p0, p1)) {
                const int buf = ACC_BUFS == 2 ? (seg & 1) : 0;
                if (seg >= ACC_BUFS) {
                    if (!tc::mbar_wait_abortable(&acc_empty[buf], (uint32_t)((seg / ACC_BUFS - 1) & 1), g.budget, &s_abort)) { ok = false; break; }
                    tc::fence_after_sync();
                }
                const uint32_t acc = tmem_base + (uint32_t)(buf * ACC_STRIDE);
                for (int p = p0; p < p1; ++it) {
                    const int gn = min(G, p1 - p);               // panels in this stage
                    const long long tw0 = prof ? clock64() : 0;
                    if (!tc::mbar_wait_abortable(&full_bar[s], full_phase, g.budget, &s_abort)) { ok = false; break; }
                    if (prof) prof_wait += clock64() - tw0;
                    tc::fence_after_sync();
                    const uint32_t st_lo = (uint32_t)s * (uint32_t)(kStage >> 4);
                    const uint32_t sf_t0 = tmem_base + SF_COL0 + (uint32_t)(it % kSfBufs) * SF_BUF_COLS;
                    const long long ts0 = prof ? clock64() : 0;
                    if constexpr (kSplitSf) {
                        // the scale factors of this stage were copied to tensor memory by warp 6
                        if (!tc::mbar_wait_abortable(&sf_ready[it % kSfBufs], (uint32_t)((it / kSfBufs) & 1), g.budget, &s_abort)) { ok = false; break; }
                        tc::fence_after_sync();
                    } else if (!(g.dbg & 1)) {
                        for (int j = 0; j < gn; ++j)
#pragma unroll
                            for (int a = 0; a < APP; ++a)
                                tc::tmem_cp_sf(sf_t0 + (uint32_t)j * SFA_COLS + 4 * a,
                                               tc::desc_pack(sfa_lo0 + st_lo + (uint32_t)(j * (kSfaBytes >> 4) + a * 32), tc::kDescSfHi));
                    }
                    const long long ts1 = prof ? clock64() : 0;
                    prof_sf += ts1 - ts0;
                    for (int j = 0; j < gn; ++j, ++pi) {
                        const uint32_t sf_t = sf_t0 + (uint32_t)j * SFA_COLS;
                        const uint32_t a_lo = a_lo0 + st_lo + (uint32_t)j * (uint32_t)(kBsATile >> 4);
                        uint32_t b_lo, sfb_t;
                        if constexpr (RES) {
                            const int slot = g.res_full ? p + j : pi;
                            b_lo = bres_lo0 + (uint32_t)slot * (uint32_t)(kBTile >> 4);
                            sfb_t = tmem_base + SFB_RES_COL0 + (uint32_t)slot * (4 * APP);
                        } else {
                            b_lo = a_lo + (uint32_t)(kOffB >> 4);
                            sfb_t = sf_t + SFA_COLS;
                        }
                        if (!(g.dbg & 4)) {
#pragma unroll
                            for (int kb = 0; kb < 4; ++kb) {
                                const uint64_t adesc = tc::desc_pack(a_lo + 2 * kb, tc::kDescSw128Hi);
                                const uint64_t bdesc = tc::desc_pack(b_lo + 2 * kb, tc::kDescSw128Hi);
                                const uint32_t accum = (p + j > p0 || kb > 0) ? 1u : 0u;
                                if constexpr (FMT == W_NVFP4) {
                                    constexpr uint32_t idesc = tc::idesc_block_scaled(128, NB, tc::kFmtE2M1_mxf4, tc::kSfUE4M3, 0, 0);
                                    tc::mma_nvfp4_ss(acc, adesc, bdesc, idesc, accum, sf_t + 4 * kb, sfb_t + 4 * NBLK * kb);
                                } else {
                                    const uint32_t idesc = tc::idesc_block_scaled(128, NB, tc::kFmtE4M3, tc::kSfUE8M0, (uint32_t)kb, (uint32_t)kb);
                                    tc::mma_mxfp8_ss(acc, adesc, bdesc, idesc, accum, sf_t, sfb_t);
                                }
                            }
                        }
                    }
                    p += gn;
                    const long long ts2 = prof ? clock64() : 0;
                    tc::mma_commit(&empty_bar[s]);
                    if constexpr (kSplitSf) tc::mma_commit(&sf_free[it % kSfBufs]);
                    if (prof) { prof_mma += ts2 - ts1; prof_commit += clock64() - ts2; }
                    if (++s == stages) { s = 0; full_phase ^= 1u; }
                }
                if (ok) tc::mma_commit(&acc_full[buf]);
                ++seg;
            }
            s_consumed = it;
            if (prof) { g.prof[6] = prof_wait; g.prof[7] = clock64(); g.prof[8] = it; g.prof[16] = prof_sf; g.prof[17] = prof_mma; g.prof[18] = prof_commit; }
            if (!ok || s_abort != 0) {
                // give MMAs already issued a bounded chance to retire before the tensor memory is freed
                tc::mma_commit(&drain_bar);
                tc::mbar_wait(&drain_bar, 0, g.budget < 4000000ll ? g.budget : 4000000ll);
            }
        }
    } else if (warp == 6) {
        // ------------------------------------------------ scale-factor copies (tcgen05.cp), ahead of the MMAs (streamed path)
        if (kSplitSf && lane == 0) {
            int it = 0, t, p0, p1, s = 0;
            uint32_t full_phase = 0;
            BsSegIter S{u0, u1, P};
            bool ok = true;
            const uint32_t sfa_lo0 = (tc::smem_u32(smem + kOffSfa) >> 4) & 0x3FFFu;
            while (ok && S.next(t, p0, p1)) {
                for (int p = p0; p < p1; ++p, ++it) {
                    // the columns of this parity are free once the MMAs of two stages ago have retired
                    if (it >= kSfBufs && !tc::mbar_wait_abortable(&sf_free[it % kSfBufs], (uint32_t)((it / kSfBufs - 1) & 1), g.budget, &s_abort)) { ok = false; break; }
                    if (!tc::mbar_wait_abortable(&full_bar[s], full_phase, g.budget, &s_abort)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t st_lo = (uint32_t)s * (uint32_t)(kStage >> 4);
                    const uint32_t sf_t = tmem_base + SF_COL0 + (uint32_t)(it % kSfBufs) * SF_BUF_COLS;
                    if (!(g.dbg & 1)) {
#pragma unroll
                        for (int a = 0; a < APP; ++a)
                            tc::tmem_cp_sf(sf_t + 4 * a, tc::desc_pack(sfa_lo0 + st_lo + (uint32_t)(a * 32), tc::kDescSfHi));
                    }
                    if constexpr (!RES) {
                        const uint32_t sfb_t = sf_t + SFA_COLS;
                        const uint32_t sfb_lo = sfa_lo0 + st_lo + (uint32_t)(kSfaBytes >> 4);
#pragma unroll
                        for (int a = 0; a < APP; ++a)
#pragma unroll
                            for (int j = 0; j < NBLK; ++j)
                                tc::tmem_cp_sf(sfb_t + 4 * (a * NBLK + j), tc::desc_pack(sfb_lo + (uint32_t)((j * APP + a) * 32), tc::kDescSfHi));
                    }
                    tc::mma_commit(&sf_ready[it % kSfBufs]);
                    if (++s == stages) { s = 0; full_phase ^= 1u; }
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------ epilogue: warps 2..5 own TMEM lane quadrant (warp % 4)
        // Control flow below depends only on values that are uniform over the 128 epilogue threads, so every
        // named barrier is reached by all of them even after a wait has run out (`ok` only gates memory work;
        // once the abort flag is up every later wait returns at once).
        const int quad = warp & 3, etid = (int)threadIdx.x - 64;
        const int row_l = quad * 32 + lane;                 // feature inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        int seg = 0, t, p0, p1;
        BsSegIter S{u0, u1, P};
        bool ok = true;
        // stores one finished value (row m, feature n) with the residual / dtype epilogue; returns what it stored
        auto store_plain = [&](int m, int n, float y) -> float {
            if (g.epilogue == EPI_RESIDUAL)
                y = bf16_to_f32(f32_to_bf16(y)) + bf16_to_f32(g.residual[(size_t)m * g.ld_res + n]);
            if (g.out_f32) { reinterpret_cast<float*>(g.out)[(size_t)m * g.ldo + n] = y; return y; }
            const __nv_bfloat16 o = f32_to_bf16(y);
            reinterpret_cast<__nv_bfloat16*>(g.out)[(size_t)m * g.ldo + n] = o;
            return bf16_to_f32(o);
        };
        long long prof_ewait = 0, prof_ework = 0;
        while (S.next(t, p0, p1)) {
            const int buf = ACC_BUFS == 2 ? (seg & 1) : 0;
            const long long te0 = prof ? clock64() : 0;
            if (!tc::mbar_wait_abortable(&acc_full[buf], (uint32_t)((seg / ACC_BUFS) & 1), g.budget, &s_abort)) ok = false;
            const long long te1 = prof ? clock64() : 0;
            prof_ewait += te1 - te0;
            ok = __all_sync(0xffffffffu, ok);           // warp-uniform: the shuffles below need every lane
            if constexpr (!RES) {
                // the streamed epilogue has named barriers inside its row-block loop: agree on `ok` across the four warps
                if (!ok) s_abort = 1;
                epi_bar_sync();
                if (etid == 0) s_ssq[1] = s_abort == 0 ? 1.f : 0.f;
                epi_bar_sync();
                ok = s_ssq[1] != 0.f;
            }
            tc::fence_after_sync();
            const uint32_t acc = tmem_base + (uint32_t)(buf * ACC_STRIDE) + lane_addr;
            const int tn = t / g.tiles_m, tm = t - tn * g.tiles_m;
            const int n = tn * kBsTileN + row_l;
            const bool complete = p0 == 0 && p1 == P;
            // Tiles cut over several CTAs: every contributor stores its raw fp32 partial and bumps the tile's counter;
            // the one that arrives last (all partials are then complete) adds them in CTA order -- the same sum
            // whoever does it -- and runs the epilogue.  Nobody waits for anybody.
            int c_first = blockIdx.x, c_last = blockIdx.x;
            bool finisher = true;
            if (!complete) {
                c_first = unit_owner(g.total_units, gridDim.x, t * P);
                c_last = unit_owner(g.total_units, gridDim.x, (t + 1) * P - 1);
                // a CTA holds at most two cut segments: the tail of one tile (slot 0) and the head of another (slot 1)
                float* wp = g.ws + (size_t)(2 * blockIdx.x + (p0 == 0 ? 1 : 0)) * (NB * 128) + row_l;
                if (ok) {
#pragma unroll 1
                    for (int c0 = 0; c0 < NB; c0 += CH) {
                        if (tm * NB + c0 >= g.M) break;             // columns of dead rows are never read back
                        uint32_t r[CH];
                        if constexpr (CH == 16) tc::tmem_ld_32x16(acc + c0, r); else tc::tmem_ld_32x32(acc + c0, r);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < CH; ++j) wp[(size_t)(c0 + j) * 128] = __uint_as_float(r[j]);
                    }
                }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
                __threadfence();
                epi_bar_sync();
                if (etid == 0) {
                    const uint32_t prev = atomicAdd(g.flags + t, 1u);
                    const bool last = prev + 1u == (uint32_t)(c_last - c_first + 1);
                    if (last) g.flags[t] = 0u;                       // ready for the next launch
                    __threadfence();
                    s_ssq[0] = last ? 1.f : 0.f;                     // broadcast through shared memory
                }
                epi_bar_sync();
                finisher = s_ssq[0] != 0.f;
                epi_bar_sync();                                      // s_ssq is reused below
            }
            if (finisher) {
                const bool tp_on = g.tp.size > 1;
                const bool staged = !RES && !g.out_f32 && !tp_on;       // bf16 output of many rows: staged through shared memory
                bool released = false;
                // the staged epilogue never forms the per-row sums, so it must not publish any (what is in s_ssq then is whatever
                // the finisher test left there)
                const bool want_ssq = g.ssq_out != nullptr && g.epilogue != EPI_SWIGLU && !staged;
                uint32_t tp_val = 0; size_t tp_par = 0;
                if (tp_on) {
                    tp_val = g.tp.counter[t] + 1u;
                    tp_par = (size_t)(tp_val & 1u) * g.tp.size * g.tp.max_rows * g.tp.n_pad;
                }
                if (ok) {
#pragma unroll 1
                    for (int c0 = 0; c0 < NB; c0 += CH) {
                        if (tm * NB + c0 >= g.M) break;             // uniform: no live row from here on
                        float v[CH];
                        if (complete) {
                            uint32_t r[CH];
                            if constexpr (CH == 16) tc::tmem_ld_32x16(acc + c0, r); else tc::tmem_ld_32x32(acc + c0, r);
                            tc::tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(r[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < CH; ++j) v[j] = 0.f;
                        }
                        // all contributors' partials (this CTA's included), a few at a time so their loads overlap;
                        // added in CTA order
                        constexpr int FB = CH == 16 ? 4 : 2;
                        for (int cb = c_first; !complete && cb <= c_last; cb += FB) {
                            float pv[FB][CH];
#pragma unroll
                            for (int u = 0; u < FB; ++u) {
                                const int cc = min(cb + u, c_last);
                                const float* pp = g.ws + (size_t)(2 * cc + (cc == c_first ? 1 : 0)) * (NB * 128) + row_l;
#pragma unroll
                                for (int j = 0; j < CH; ++j) pv[u][j] = __ldcg(pp + (size_t)(c0 + j) * 128);
                            }
#pragma unroll
                            for (int u = 0; u < FB; ++u) {
                                if (cb + u <= c_last) {
#pragma unroll
                                    for (int j = 0; j < CH; ++j) v[j] += pv[u][j];
                                }
                            }
                        }
                        // the row factors of the chunk sit one per lane and are broadcast with a shuffle
                        const int m_base = tm * NB + c0;
                        float rs_lane = g.out_scale;
                        if constexpr (RES) rs_lane *= s_inv_rms[(c0 + lane) & 31];
                        else if (g.row_scale != nullptr && m_base + lane < g.M) rs_lane *= g.row_scale[m_base + lane];
                        if (staged) {
                            // lean bodies, one per epilogue kind (no per-element mode branches): values go to the staging
                            // block as rows of 128 (64 after SwiGLU) bf16; rows past M are staged too and never written out
                            __nv_bfloat16* srow = sEpi + (c0 & 127) * (g.epilogue == EPI_SWIGLU ? 64 : 128);
                            if (g.epilogue == EPI_SWIGLU) {
#pragma unroll
                                for (int j = 0; j < CH; ++j) {
                                    const float yb = bf16_to_f32(f32_to_bf16(v[j] * __shfl_sync(0xffffffffu, rs_lane, j & 31)));
                                    const float other = __shfl_xor_sync(0xffffffffu, yb, 1);
                                    const float o = __fdividef(yb, 1.f + __expf(-yb)) * other;
                                    if (!(lane & 1)) srow[j * 64 + (row_l >> 1)] = f32_to_bf16(o);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < CH; ++j)
                                    srow[j * 128 + row_l] = f32_to_bf16(v[j] * __shfl_sync(0xffffffffu, rs_lane, j & 31));
                            }
                        } else {
                        float resv[CH];
                        const bool use_res = g.epilogue == EPI_RESIDUAL && !tp_on;
#pragma unroll
                        for (int j = 0; j < CH; ++j)
                            resv[j] = (use_res && m_base + j < g.M && n < g.N) ? bf16_to_f32(g.residual[(size_t)(m_base + j) * g.ld_res + n]) : 0.f;
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            const int m = m_base + j;
                            const float y = v[j] * __shfl_sync(0xffffffffu, rs_lane, j & 31);
                            if (m >= g.M) continue;                 // uniform over the warp
                            if (tp_on) {
                                // tensor-parallel combine, step 1: push this rank's partial into every rank's receive buffer
                                if (n < g.N) {
                                    const size_t off = tp_par + ((size_t)g.tp.rank * g.tp.max_rows + m) * g.tp.n_pad + n;
                                    for (int pr = 0; pr < g.tp.size; ++pr) g.tp.recv[pr][off] = y;
                                }
                            } else if (g.epilogue == EPI_SWIGLU) {
                                const float yb = bf16_to_f32(f32_to_bf16(y));
                                const float other = __shfl_xor_sync(0xffffffffu, yb, 1);
                                if (!(lane & 1) && n + 1 < g.N) {
                                    const float o = __fdividef(yb, 1.f + __expf(-yb)) * other;
                                    if (g.out_f32) reinterpret_cast<float*>(g.out)[(size_t)m * g.ldo + (n >> 1)] = o;
                                    else reinterpret_cast<__nv_bfloat16*>(g.out)[(size_t)m * g.ldo + (n >> 1)] = f32_to_bf16(o);
                                }
                            } else {
                                float o = 0.f;
                                if (n < g.N) {
                                    float yy = y;
                                    if (use_res) yy = bf16_to_f32(f32_to_bf16(y)) + resv[j];
                                    if (g.out_f32) { reinterpret_cast<float*>(g.out)[(size_t)m * g.ldo + n] = yy; o = yy; }
                                    else {
                                        const __nv_bfloat16 ob = f32_to_bf16(yy);
                                        reinterpret_cast<__nv_bfloat16*>(g.out)[(size_t)m * g.ldo + n] = ob;
                                        o = bf16_to_f32(ob);
                                    }
                                }
                                if (want_ssq && c0 + j < 32) {
                                    const float sq = warp_sum(o * o);
                                    if (lane == 0) s_ssq[quad * 32 + c0 + j] = sq;
                                }
                            }
                        }
                        }
                        if (staged && (((c0 + CH) & 127) == 0 || c0 + CH >= NB || tm * NB + c0 + CH >= g.M)) {
                            // a block of up to 128 batch rows is staged: release the accumulator if it was the last one,
                            // then write the rows out (and add the residual) in 16-byte pieces, full row segments per warp
                            const int rb0 = tm * NB + ((c0 + CH - 1) & ~127);
                            const bool last_block = c0 + CH >= NB || tm * NB + c0 + CH >= g.M;
                            if (last_block && complete) {
                                tc::fence_before_sync();
                                __syncwarp();
                                if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
                                released = true;
                            }
                            epi_bar_sync();
                            const int cols = g.epilogue == EPI_SWIGLU ? 64 : 128, cpr = cols >> 3;
                            const int n_base = g.epilogue == EPI_SWIGLU ? (tn * kBsTileN) >> 1 : tn * kBsTileN;
                            const int n_lim = g.epilogue == EPI_SWIGLU ? g.N >> 1 : g.N;
                            const int rcnt = min(128, g.M - rb0);
                            __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(g.out);
                            for (int i = etid; i < rcnt * cpr; i += 128) {
                                const int rr = i / cpr, ch = i - rr * cpr;
                                const int m = rb0 + rr, n0 = n_base + ch * 8;
                                if (n0 >= n_lim) continue;
                                const uint4 sv = *reinterpret_cast<const uint4*>(sEpi + rr * cols + ch * 8);
                                uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
                                __nv_bfloat16* dst = outp + (size_t)m * g.ldo + n0;
                                if (g.rs.size > 1) {
                                    // tensor parallel: the piece goes to the rank that owns row m (peer store)
                                    const int owner = m / g.rs.rpr;
                                    dst = g.rs.recv[owner] + ((size_t)g.rs.rank * g.rs.rpr + (m - owner * g.rs.rpr)) * g.rs.ld + n0;
                                }
                                const bool full = n0 + 8 <= n_lim;
                                if (g.epilogue == EPI_RESIDUAL) {
                                    const __nv_bfloat16* rp = g.residual + (size_t)m * g.ld_res + n0;
                                    if (full && (reinterpret_cast<uintptr_t>(rp) & 15) == 0) {
                                        const uint4 rv = *reinterpret_cast<const uint4*>(rp);
                                        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            const float2 a2 = bf16x2_bits_to_f32x2(w[e]), r2 = bf16x2_bits_to_f32x2(rw[e]);
                                            w[e] = f32x2_to_bf16x2_bits(a2.x + r2.x, a2.y + r2.y);
                                        }
                                    } else {
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            const float2 a2 = bf16x2_bits_to_f32x2(w[e]);
                                            const float r0 = n0 + 2 * e < n_lim ? bf16_to_f32(rp[2 * e]) : 0.f;
                                            const float r1 = n0 + 2 * e + 1 < n_lim ? bf16_to_f32(rp[2 * e + 1]) : 0.f;
                                            w[e] = f32x2_to_bf16x2_bits(a2.x + r0, a2.y + r1);
                                        }
                                    }
                                }
                                if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                                } else {
#pragma unroll
                                    for (int e = 0; e < 8; ++e)
                                        if (n0 + e < n_lim) dst[e] = reinterpret_cast<const __nv_bfloat16*>(w)[e];
                                }
                            }
                            epi_bar_sync();             // the staging block is free again
                        }
                    }
                }
                if (complete && !released) {
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
                }
                if (tp_on) {
                    // step 2: publish (one system-scope release per peer, cumulative over the stores ordered by the
                    // barrier), step 3: wait (bounded) for the same tile of every peer
                    epi_bar_sync();
                    if (etid < g.tp.size && s_abort == 0) {
                        uint32_t* f = g.tp.flags[etid] + (size_t)t * g.tp.size + g.tp.rank;
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(tp_val) : "memory");
                        const uint32_t* mine = g.tp.flags[g.tp.rank] + (size_t)t * g.tp.size + etid;
                        const long long t0 = clock64();
                        uint32_t seen;
                        do {
                            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
                            if ((int32_t)(seen - tp_val) >= 0) break;
                            if (clock64() - t0 > g.budget) { s_abort = 1; break; }
                        } while (true);
                    }
                    epi_bar_sync();
                    if (s_abort != 0) ok = false;
                    if (etid == 0 && ok) g.tp.counter[t] = tp_val;
                    if (ok) {
                        // step 4: add the ranks' partials in rank order (identical everywhere), then the epilogue
                        const float* rbuf = g.tp.recv[g.tp.rank] + tp_par;
                        for (int mm = 0; mm < NB; ++mm) {
                            const int m = tm * NB + mm;
                            if (m >= g.M) break;
                            float y = 0.f;
                            if (n < g.N)
                                for (int pr = 0; pr < g.tp.size; ++pr) y += __ldcv(rbuf + ((size_t)pr * g.tp.max_rows + m) * g.tp.n_pad + n);
                            const float o = n < g.N ? store_plain(m, n, y) : 0.f;
                            if (want_ssq && mm < 32) {
                                const float sq = warp_sum(o * o);
                                if (lane == 0) s_ssq[quad * 32 + mm] = sq;
                            }
                        }
                    }
                }
                if (want_ssq) {
                    // partial sums of squares of the stored rows over this tile's 128 features, quadrants added in order
                    epi_bar_sync();
                    const int m = tm * NB + etid;
                    if (etid < 32 && etid < NB && m < g.M && ok)
                        g.ssq_out[(size_t)m * g.ssq_out_ld + tn] = s_ssq[etid] + s_ssq[32 + etid] + s_ssq[64 + etid] + s_ssq[96 + etid];
                    epi_bar_sync();             // s_ssq is reused by the next tile
                }
            }
            ++seg;
            if (prof) prof_ework += clock64() - te1;
        }
        if (prof && etid == 0) { g.prof[9] = clock64(); g.prof[11] = prof_ewait; g.prof[12] = prof_ework; g.prof[13] = seg; }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (prof && threadIdx.x == 0) g.prof[10] = clock64();
    if (s_abort != 0 && threadIdx.x == 0) {
        set_status(g.status, PS_DEV_WAIT_TIMEOUT);
        // copies still in flight get a bounded chance to land before the shared memory goes away
        const long long b = g.budget < 4000000ll ? g.budget : 4000000ll;
        for (int c = s_consumed; c < s_issued; ++c) tc::mbar_wait(&full_bar[c % stages], (uint32_t)((c / stages) & 1), b);
    }
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

// ---- stand-alone activation quantiser for the streamed path: one CTA per row.  Quantises x (1 + w) and leaves the
// row factor 1/rms in `row_scale` for the projection's epilogue (same split of the RMSNorm as the resident prologue).
template <int FMT>
__global__ void __launch_bounds__(256) act_quant_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int M, int K, int P,
                                                        const __nv_bfloat16* __restrict__ norm_w, float eps, float c1, float gs,
                                                        uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
                                                        float* __restrict__ row_scale) {
    using T = BsT<FMT>;
    __shared__ float red[32];
    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();
    const int m = blockIdx.x;
    const __nv_bfloat16* xr = x + (size_t)m * ldx;
    if (row_scale != nullptr) {
        float inv_rms = 1.f;
        if (norm_w != nullptr) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < (K >> 3); i += 256) {
                const uint4 xv = reinterpret_cast<const uint4*>(xr)[i];
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 a = bf16x2_bits_to_f32x2(xw[e]); ss += a.x * a.x + a.y * a.y; }
            }
            ss = block_sum(ss, red);
            inv_rms = rsqrtf(ss / (float)K + eps);
        }
        if (threadIdx.x == 0) row_scale[m] = inv_rms;
    }
    uint8_t* crow = codes + (size_t)m * P * 128;
    uint8_t* atoms = sf + (size_t)(m >> 7) * P * T::kApp * 512;
    const int rr = m & 127;
    constexpr int NVEC = T::kBlockK / 8;
    for (int b = threadIdx.x; b < P * T::kBpp; b += 256) {
        const int p = b / T::kBpp, blk = b % T::kBpp;
        const int k0 = p * T::kPanelK + blk * T::kBlockK;
        float v[T::kBlockK];
#pragma unroll
        for (int v4 = 0; v4 < NVEC; ++v4) {
            const bool in = k0 + v4 * 8 < K;
            const uint4 xv = in ? *reinterpret_cast<const uint4*>(xr + k0 + v4 * 8) : make_uint4(0, 0, 0, 0);
            const uint4 wv = (in && norm_w != nullptr) ? __ldg(reinterpret_cast<const uint4*>(norm_w + k0 + v4 * 8)) : make_uint4(0, 0, 0, 0);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a2 = bf16x2_bits_to_f32x2(xw[e]), w2 = bf16x2_bits_to_f32x2(ww[e]);
                v[v4 * 8 + 2 * e] = __fmul_rn(a2.x, 1.f + w2.x);
                v[v4 * 8 + 2 * e + 1] = __fmul_rn(a2.y, 1.f + w2.y);
            }
        }
        if constexpr (FMT == W_NVFP4) {
            uint2 c; uint8_t s;
            quant_block_nvfp4(v, c1, gs, c, s);
            *reinterpret_cast<uint2*>(crow + (size_t)p * 128 + blk * 8) = c;
            atoms[((size_t)p * 4 + (blk >> 2)) * 512 + sf_atom_off(rr, blk & 3)] = s;
        } else {
            uint4 c[2]; uint8_t s;
            quant_block_mxfp8(v, c, s);
            uint4* d = reinterpret_cast<uint4*>(crow + (size_t)p * 128 + blk * 32);
            d[0] = c[0]; d[1] = c[1];
            atoms[(size_t)p * 512 + sf_atom_off(rr, blk)] = s;
        }
    }
}

typedef CUresult (*BsEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static BsEncodeTiledFn bs_encode_fn() {
    static BsEncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<BsEncodeTiledFn>(p);
    }
    return fn;
}

// Byte matrix [rows, row_bytes] (pitch `pitch` bytes) with a (box_rows x 128 byte) box and 128-byte swizzle.
static int bs_make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch, uint32_t box_rows) {
    BsEncodeTiledFn enc = bs_encode_fn();
    if (enc == nullptr) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {128u, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static long long* g_bs_prof = nullptr;
static int g_bs_prof_skip = 0;
static int g_bs_sms = 0;
static int bs_sm_count() {
    if (g_bs_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_bs_sms, cudaDevAttrMultiProcessorCount, dev);
        const char* e = getenv("PS_BS_GRID");          // tests: emulate another SM count
        if (e != nullptr && atoi(e) > 0) g_bs_sms = atoi(e);
    }
    return g_bs_sms;
}

constexpr int kBsMinUnits = 4;
struct BsPlan { int P, tiles_n, tiles_m, total, grid, stages, res_slots, res_full, nb; size_t smem; };

template <int FMT>
static bool bs_plan(int M, int N, int K, bool resident, int grid_override, BsPlan& pl) {
    using T = BsT<FMT>;
    pl.P = (K + T::kPanelK - 1) / T::kPanelK;
    pl.tiles_n = (N + kBsTileN - 1) / kBsTileN;
    pl.nb = resident ? (M <= 16 ? 16 : 32) : (M <= 128 ? 128 : 256);
    pl.tiles_m = (M + pl.nb - 1) / pl.nb;
    if ((long long)pl.tiles_n * pl.tiles_m > kBsMaxTiles) return false;
    pl.total = pl.tiles_n * pl.tiles_m * pl.P;
    const int sms = grid_override > 0 ? grid_override : bs_sm_count();
    // small projections: at least kBsMinUnits panels per CTA, so that a tile is never cut into dozens of partials
    // that its last contributor then has to sum
    const int want = (pl.total + kBsMinUnits - 1) / kBsMinUnits;
    pl.grid = want < sms ? want : sms;
    const int nblk = pl.nb > 128 ? 2 : 1;
    const int sfa = T::kApp * 512;
    const int grp = resident ? bs_group<true>() : 1;
    int stage = resident ? grp * (kBsATile + sfa) : (kBsATile + pl.nb * 128 + sfa + nblk * sfa);
    stage = (stage + 1023) / 1024 * 1024;
    size_t res_bytes = 0;
    pl.res_slots = 0; pl.res_full = 0;
    if (resident) {
        if (pl.tiles_m != 1) return false;
        const int base = pl.total / pl.grid, umax = base + (pl.total % pl.grid ? 1 : 0);
        pl.res_full = base >= pl.P ? 1 : 0;
        pl.res_slots = pl.res_full ? pl.P : umax;
        res_bytes = (size_t)pl.res_slots * (pl.nb * 128 + T::kApp * 128);
        if (64 + 2 * grp * T::kApp * 4 + pl.res_slots * T::kApp * 4 > 512) return false;   // accumulators + 2 scale sets + resident scale columns
    }
    if (!resident) res_bytes = 128 * 128 * 2;          // output staging block of the streamed path's epilogue
    const size_t avail = kBsSmemBudget - 1024;
    if (res_bytes + 3 * (size_t)stage > avail) return false;
    pl.stages = (int)((avail - res_bytes) / stage);
    if (pl.stages > kBsMaxStages) pl.stages = kBsMaxStages;
    pl.smem = res_bytes + (size_t)pl.stages * stage + 1024;
    return true;
}

template <int FMT, int NB, bool RES>
static int bs_launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mn, const BsArgs& a, const BsPlan& pl,
                     cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_bs_kernel<FMT, NB, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBsSmemBudget);
        attr_set = true;
    }
    return launch_pdl(gemm_bs_kernel<FMT, NB, RES>, dim3(pl.grid), dim3(bs_threads<RES>()), pl.smem, stream, mw, mx, mn, a);
}

template <int FMT>
static int bs_dispatch(const void* w_codes, long long w_row_bytes, long long w_pitch, const void* xq_codes, BsArgs& a,
                       bool resident, int grid_override, const CUtensorMap* map_next, cudaStream_t stream) {
    BsPlan pl;
    if (!bs_plan<FMT>(a.M, a.N, a.K, resident, grid_override, pl)) return -1;
    a.P = pl.P; a.tiles_n = pl.tiles_n; a.tiles_m = pl.tiles_m; a.total_units = pl.total; a.stages = pl.stages;
    a.res_slots = pl.res_slots; a.res_full = pl.res_full;
    CUtensorMap mw, mx;
    int err = bs_make_map(&mw, w_codes, (uint64_t)a.N, (uint64_t)w_row_bytes, (uint64_t)w_pitch, kBsTileN);
    if (err) return err;
    if (!resident) {
        err = bs_make_map(&mx, xq_codes, (uint64_t)a.M, (uint64_t)pl.P * 128, (uint64_t)pl.P * 128, (uint32_t)pl.nb);
        if (err) return err;
    } else {
        mx = mw;
    }
    const CUtensorMap& mn = map_next != nullptr ? *map_next : mw;
    if (map_next == nullptr) a.next_total = 0;
    if (resident) return pl.nb == 16 ? bs_launch<FMT, 16, true>(mw, mx, mn, a, pl, stream) : bs_launch<FMT, 32, true>(mw, mx, mn, a, pl, stream);
    return pl.nb == 128 ? bs_launch<FMT, 128, false>(mw, mx, mn, a, pl, stream) : bs_launch<FMT, 256, false>(mw, mx, mn, a, pl, stream);
}

}  // namespace ps

// Query the launch plan: fills out[8] = {grid, stages, resident slots, NB, panels per tile, tiles_n, tiles_m,
// dynamic shared memory}; returns 1 when the (resident or streamed) path can run this shape, else 0.
PS_API int ps_gemm_bs_plan(int wfmt, int M, int N, int K, int resident, int grid_override, int* out) {
    using namespace ps;
    BsPlan pl;
    bool ok = false;
    if (wfmt == W_NVFP4) ok = bs_plan<W_NVFP4>(M, N, K, resident != 0, grid_override, pl);
    else if (wfmt == W_MXFP8) ok = bs_plan<W_MXFP8>(M, N, K, resident != 0, grid_override, pl);
    if (!ok) return 0;
    out[0] = pl.grid; out[1] = pl.stages; out[2] = pl.res_slots; out[3] = pl.nb; out[4] = pl.P; out[5] = pl.tiles_n;
    out[6] = pl.tiles_m; out[7] = (int)pl.smem;
    return 1;
}

// Development aid: CTA 0 of later launches writes clock64() stamps of its phases into `buf` (32 x int64 on the
// device): [0] start, [1] set-up done, [2] stream predecessor done, [3] row statistics done, [4] quantisation done,
// [5] prologue barrier, [6] cycles the MMA thread waited for data, [7] MMA thread done, [8] stages, [9] epilogue
// done, [10] end.  Only the launch after `skip_launches` further ones is stamped (also inside a graph capture).
// Pass null to stop.
PS_API void ps_gemm_bs_profile(void* buf, int skip_launches) { ps::g_bs_prof = (long long*)buf; ps::g_bs_prof_skip = skip_launches; }

// Bytes of stream-K workspace (partials) and number of flag words a launch may touch on this device.
PS_API long long ps_gemm_bs_workspace_bytes() { return (long long)ps::bs_sm_count() * 2 * 256 * 128 * 4; }
PS_API int ps_gemm_bs_flag_words() { return ps::kBsMaxTiles; }

// out = epilogue( act . W^T ) on the block-scaled tensor-core path.
//   w_codes [N rows, pitch w_pitch bytes] canonical codes, w_sf = scale atoms [ceil(N/128)][P * app][512]
//   resident path (xq_codes == null, M <= 32): x bf16 [M, ldx], optional fused RMSNorm(1 + norm_w) whose row sums
//     of squares are `ssq_n` partials per row at ssq_in (null: the kernel sweeps the rows itself)
//   streamed path: xq_codes [M, P * 128], xq_sf atoms and row_scale [M] from ps_act_quant (same act_gs)
//   next_*: optionally the weights of the projection that will run next with the same rows; their first bytes are
//     prefetched into L2 while this one drains
//   ssq_out (M <= 32, store / residual epilogue): receives one partial sum of squares of the stored values per row
//     and 128-feature tile, [M][ssq_out_ld]
// Returns a cudaError_t value, or -1 (nothing launched) when the requested path cannot hold the shape.
PS_API int ps_gemm_bs(int wfmt, const void* w_codes, long long w_row_bytes, long long w_pitch, const void* w_sf,
                      float w_tscale, int M, int N, int K, const void* x, int ldx, const void* norm_w, float eps,
                      float act_gs, void* xn_out, const void* ssq_in, int ssq_n, int ssq_in_ld, void* ssq_out,
                      int ssq_out_ld, const void* xq_codes, const void* xq_sf, const void* row_scale, int epilogue,
                      const void* residual, int ld_res, void* out, int ldo, int out_f32, void* ws, void* flags,
                      const void* tp_combine, void* status, int grid_override, int next_fmt, const void* next_codes,
                      long long next_row_bytes, long long next_pitch, const void* next_sf, int next_N, int next_K,
                      const void* tp_scatter, cudaStream_t stream) {
    using namespace ps;
    if (M < 1 || N < 1 || K < 8 || (K % 8) || ((uintptr_t)w_codes % 16) || (w_pitch % 16) || ((uintptr_t)w_sf % 16))
        return (int)cudaErrorInvalidValue;
    const bool resident = xq_codes == nullptr;
    if (resident && (x == nullptr || (ldx % 8) || ((uintptr_t)x % 16) || M > 32)) return (int)cudaErrorInvalidValue;
    if (!resident && (xq_sf == nullptr || ((uintptr_t)xq_codes % 16) || ((uintptr_t)xq_sf % 16))) return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && (N & 1)) return (int)cudaErrorInvalidValue;
    if (ws == nullptr || flags == nullptr) return (int)cudaErrorInvalidValue;
    BsArgs a;
    a.M = M; a.N = N; a.K = K;
    a.sfw = (const uint8_t*)w_sf;
    const bool nv = wfmt == W_NVFP4;
    a.out_scale = nv ? w_tscale * act_gs : w_tscale;
    a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps;
    a.act_gs = act_gs; a.act_c1 = 1.0f / (6.0f * act_gs);
    a.xn_out = (__nv_bfloat16*)xn_out;
    a.ssq_in = (const float*)ssq_in; a.ssq_n = ssq_n; a.ssq_in_ld = ssq_in_ld;
    a.ssq_out = M <= 32 ? (float*)ssq_out : nullptr; a.ssq_out_ld = ssq_out_ld;
    a.row_scale = (const float*)row_scale;
    a.sfx = (const uint8_t*)xq_sf;
    a.epilogue = epilogue; a.residual = (const __nv_bfloat16*)residual; a.ld_res = ld_res;
    a.out = out; a.ldo = ldo; a.out_f32 = out_f32;
    a.ws = (float*)ws; a.flags = (uint32_t*)flags; a.status = (uint32_t*)status; a.budget = g_ps_wait_budget_cycles;
    { const char* e = getenv("PS_BS_DBG"); a.dbg = e != nullptr ? atoi(e) : 0; }
    a.prof = nullptr;
    if (g_bs_prof != nullptr && g_bs_prof_skip-- == 0) a.prof = g_bs_prof;
    if (tp_combine != nullptr) {
        a.tp = *reinterpret_cast<const TpCombine*>(tp_combine);
        if (a.tp.size > kTpMaxRanks || M > a.tp.max_rows || N > a.tp.n_pad || epilogue == EPI_SWIGLU)
            return (int)cudaErrorInvalidValue;
    } else {
        a.tp.size = 0;
    }
    a.rs.size = 0;
    if (tp_scatter != nullptr) {
        a.rs = *reinterpret_cast<const TpScatter*>(tp_scatter);
        // only the streamed path's staged bf16 store knows how to scatter
        if (a.rs.size > kTpMaxRanks || resident || epilogue != EPI_STORE || out_f32 || tp_combine != nullptr || (a.rs.ld % 8) ||
            a.rs.rpr < 1 || (long long)a.rs.rpr * a.rs.size < M || N > a.rs.ld)
            return (int)cudaErrorInvalidValue;
    }
    // the projection that runs next with the same number of rows: geometry of its first ring fill, for the L2 prefetch
    CUtensorMap map_next;
    const CUtensorMap* mnp = nullptr;
    a.next_total = 0;
    if (next_codes != nullptr && next_sf != nullptr && (next_fmt == W_NVFP4 || next_fmt == W_MXFP8)) {
        BsPlan np;
        const bool okp = next_fmt == W_NVFP4 ? bs_plan<W_NVFP4>(M, next_N, next_K, resident, grid_override, np)
                                             : bs_plan<W_MXFP8>(M, next_N, next_K, resident, grid_override, np);
        if (okp && bs_make_map(&map_next, next_codes, (uint64_t)next_N, (uint64_t)next_row_bytes, (uint64_t)next_pitch, kBsTileN) == 0) {
            mnp = &map_next;
            a.next_sfw = (const uint8_t*)next_sf; a.next_P = np.P; a.next_tiles_m = np.tiles_m; a.next_total = np.total;
            a.next_grid = np.grid; a.next_stages = np.stages; a.next_sf_bytes = (next_fmt == W_NVFP4 ? 4 : 1) * 512;
        }
    }
    if (nv) return bs_dispatch<W_NVFP4>(w_codes, w_row_bytes, w_pitch, xq_codes, a, resident, grid_override, mnp, stream);
    if (wfmt == W_MXFP8) return bs_dispatch<W_MXFP8>(w_codes, w_row_bytes, w_pitch, xq_codes, a, resident, grid_override, mnp, stream);
    return (int)cudaErrorInvalidValue;
}

// Quantise x (1 + norm_w) for the streamed path: codes [M, P * 128] row-major, scale atoms [ceil(M/128)][P * app][512],
// row_scale [M] = 1/rms of the raw rows (1 without a norm).
PS_API int ps_act_quant(int wfmt, const void* x, int ldx, int M, int K, const void* norm_w, float eps, float act_gs,
                        void* codes, void* sf, void* row_scale, cudaStream_t stream) {
    using namespace ps;
    if (M < 1 || K < 8 || (K % 8) || (ldx % 8) || ((uintptr_t)x % 16) || ((uintptr_t)codes % 16)) return (int)cudaErrorInvalidValue;
    const float c1 = 1.0f / (6.0f * act_gs);
    if (wfmt == W_NVFP4) {
        const int P = (K + 255) / 256;
        return launch_pdl(act_quant_kernel<W_NVFP4>, dim3(M), dim3(256), 0, stream, (const __nv_bfloat16*)x, ldx, M, K, P,
                          (const __nv_bfloat16*)norm_w, eps, c1, act_gs, (uint8_t*)codes, (uint8_t*)sf, (float*)row_scale);
    }
    if (wfmt == W_MXFP8) {
        const int P = (K + 127) / 128;
        return launch_pdl(act_quant_kernel<W_MXFP8>, dim3(M), dim3(256), 0, stream, (const __nv_bfloat16*)x, ldx, M, K, P,
                          (const __nv_bfloat16*)norm_w, eps, c1, act_gs, (uint8_t*)codes, (uint8_t*)sf, (float*)row_scale);
    }
    return (int)cudaErrorInvalidValue;
}
