// Batched-decode GEMM (2 <= M <= 64 rows) on resident bf16 weights: out[M,N] = epilogue(A[M,K] . W[N,K]^T).
//
// In this regime the problem is a stream over W.  The operands are swapped relative to the prefill GEMM:
// 128 WEIGHT rows are the M side of `tcgen05.mma` and the few batch rows the N side (16, 32 or 64), so every
// byte a TMA stage brings into shared memory is weight data (16 KB per stage, ~100 KB in flight per CTA, two
// CTAs per SM).  K is split across CTAs so that even N = 5120 yields a few hundred CTAs; each writes fp32
// partial sums [split, M, N] and a second tiny kernel adds the splits in a fixed order (deterministic) and
// applies the residual / SwiGLU / dtype epilogue.  Accumulators live in tensor memory; epilogue warps read
// them with `tcgen05.ld` (lane = weight row, column = batch row), so the partial stores are coalesced.
// All mbarrier waits are bounded; a timeout sets PS_DEV_WAIT_TIMEOUT, frees the tensor memory and returns.
//
// The reference serves this regime with its RowBlock2/4/8 WMMA kernels (src/phaseshift/models/qwen35/
// kernels/optimized/linear/psq4.hip:221-349); here it runs from a bf16 expansion that 180 GB of HBM can
// afford to keep resident next to the block-quantised weights.
#include "ps_tcgen05.cuh"

namespace ps {

constexpr int kSmBM = 128, kSmBK = 64, kSmThreads = 192;

struct SmallMArgs {
    int M, N, K;
    int nb;                 // MMA N: batch rows padded to 16 / 32 / 64
    int x_box_rows;         // rows fetched per X tile (multiple of 8)
    int iters_per_split;    // k-iterations (of 64) per split
    int splits;
    float* partial;         // [splits, M, N] fp32
    uint32_t* status;
    long long budget;       // clock-cycle budget of every mbarrier wait
};

template <int STAGES>
__global__ void __launch_bounds__(kSmThreads, 2)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const SmallMArgs g) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int kWBytes = kSmBM * kSmBK * 2;                 // 16 KB of weights per stage
    const int x_tile_bytes = g.nb * kSmBK * 2;                  // smem footprint of the X tile (all nb rows)
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sW = smem;
    unsigned char* sX = smem + STAGES * kWBytes;                // each X stage is 64 rows x 128 B = 8 KB apart
    constexpr int kXStride = 64 * kSmBK * 2;
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_abort, s_issued, s_consumed;      // stages handed to TMA / waited for by the MMA thread

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, split = blockIdx.y;
    const int total_iters = (g.K + kSmBK - 1) / kSmBK;
    const int it0 = split * g.iters_per_split;
    const int k_iters = min(g.iters_per_split, total_iters - it0);
    const int x_bytes = g.x_box_rows * kSmBK * 2;

    // rows of the X tile beyond the fetched box must read as zero
    for (int i = threadIdx.x; i < STAGES * kXStride / 16; i += kSmThreads) reinterpret_cast<uint4*>(sX)[i] = make_uint4(0, 0, 0, 0);
    tc::fence_proxy_async_smem();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full_bar[s], 1); tc::mbar_init(&empty_bar[s], 1); }
        tc::mbar_init(&acc_bar, 1);
        tc::fence_barrier_init();
        s_abort = 0; s_issued = 0; s_consumed = 0;
        tc::tma_prefetch_desc(&map_w);
        tc::tma_prefetch_desc(&map_x);
    }
    if (warp == 1) {
        tc::tmem_alloc(&tmem_base_slot, 64);        // up to 64 fp32 columns x 128 lanes
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_acc = tmem_base_slot;
    (void)x_tile_bytes;

    if (warp == 0) {
        if (lane == 0 && k_iters > 0) {
            for (int it = 0; it < k_iters; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (it >= STAGES && !tc::mbar_wait(&empty_bar[s], ph ^ 1u, g.budget)) { atomicExch(&s_abort, 1); break; }
                tc::mbar_expect_tx(&full_bar[s], kWBytes + x_bytes);
                tc::tma_load_2d(sW + s * kWBytes, &map_w, (it0 + it) * kSmBK, tile_n * kSmBM, &full_bar[s]);
                tc::tma_load_2d(sX + s * kXStride, &map_x, (it0 + it) * kSmBK, 0, &full_bar[s]);
                s_issued = it + 1;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_bf16_f32(kSmBM, g.nb);
            bool ok = true;
            for (int it = 0; it < k_iters && ok; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!tc::mbar_wait(&full_bar[s], ph, g.budget)) { atomicExch(&s_abort, 1); ok = false; break; }
                s_consumed = it + 1;
                tc::fence_after_sync();
                const uint32_t w_addr = tc::smem_u32(sW + s * kWBytes), x_addr = tc::smem_u32(sX + s * kXStride);
#pragma unroll
                for (int kk = 0; kk < kSmBK / 16; ++kk)
                    tc::mma_bf16_ss(tmem_acc, tc::smem_desc_sw128(w_addr + kk * 32), tc::smem_desc_sw128(x_addr + kk * 32), idesc,
                                    (it > 0 || kk > 0) ? 1u : 0u);
                tc::mma_commit(&empty_bar[s]);
            }
            tc::mma_commit(&acc_bar);
        }
    } else {
        // epilogue warps 2..5 -> TMEM lane quadrant (warp % 4); lane = weight row, column = batch row
        const int quad = warp & 3;
        const bool done = k_iters > 0 ? tc::mbar_wait(&acc_bar, 0, g.budget) : true;
        tc::fence_after_sync();
        const int n = tile_n * kSmBM + quad * 32 + lane;
        if (done && s_abort == 0) {
            float* dst = g.partial + (size_t)split * g.M * g.N;
            for (int c0 = 0; c0 < g.nb; c0 += 32) {
                uint32_t r[32];
                if (k_iters > 0) {
                    tc::tmem_ld_32x32(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;
                }
                if (n < g.N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < g.M) dst[(size_t)(c0 + j) * g.N + n] = __uint_as_float(r[j]);
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (s_abort != 0 && threadIdx.x == 0) {
        set_status(g.status, PS_DEV_WAIT_TIMEOUT);
        // copies still in flight get a bounded chance to land before the shared memory goes back to the next CTA
        const long long b = g.budget < 4000000ll ? g.budget : 4000000ll;
        for (int c = s_consumed; c < s_issued; ++c) tc::mbar_wait(&full_bar[c % STAGES], (uint32_t)((c / STAGES) & 1), b);
    }
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_acc, 64);
    }
}

struct SmallMReduceArgs {
    const float* partial; int splits, M, N;
    int epilogue;            // 0 store, 1 residual, 2 SwiGLU on interleaved (gate, up) columns
    const __nv_bfloat16* residual; int ld_res;
    void* out; int ldo; int out_f32;
};

// One thread per output pair (two neighbouring columns); splits are added in ascending order.
__global__ void gemm_smallm_reduce_kernel(const SmallMReduceArgs a) {
    const int pairs = a.N >> 1;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (long long)a.M * pairs) return;
    const int m = (int)(id / pairs), c = (int)(id % pairs) * 2;
    float v0 = 0.f, v1 = 0.f;
    for (int s = 0; s < a.splits; ++s) {
        const float2 p = *reinterpret_cast<const float2*>(a.partial + ((size_t)s * a.M + m) * a.N + c);
        v0 += p.x; v1 += p.y;
    }
    if (a.epilogue == 2) {
        const float gt = bf16_to_f32(f32_to_bf16(v0)), up = bf16_to_f32(f32_to_bf16(v1));
        reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + (c >> 1)] = f32_to_bf16(silu_f(gt) * up);
        return;
    }
    if (a.epilogue == 1) {
        const float2 rs = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a.residual + (size_t)m * a.ld_res + c));
        v0 = bf16_to_f32(f32_to_bf16(v0)) + rs.x;
        v1 = bf16_to_f32(f32_to_bf16(v1)) + rs.y;
    }
    if (a.out_f32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + (size_t)m * a.ldo + c) = make_float2(v0, v1);
    else *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)m * a.ldo + c) = f32x2_to_bf16x2_bits(v0, v1);
}

typedef CUresult (*SmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static SmEncodeFn sm_encode_fn() {
    static SmEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<SmEncodeFn>(p);
    }
    return fn;
}

static int sm_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    SmEncodeFn enc = sm_encode_fn();
    if (enc == nullptr) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kSmBK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace ps

// Number of K splits the launcher will use (the caller sizes `partial` = splits * M * N floats with it).
PS_API int ps_gemm_smallm_splits(int N, int K) {
    const int tiles = (N + ps::kSmBM - 1) / ps::kSmBM;
    const int iters = (K + ps::kSmBK - 1) / ps::kSmBK;
    int splits = (296 + tiles - 1) / tiles;                 // two CTAs on each of 148 SMs
    const int max_splits = iters / 8 > 0 ? iters / 8 : 1;   // at least 8 k-iterations (128 KB of weights) per CTA
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 16) splits = 16;
    const int per = (iters + splits - 1) / splits;
    return (iters + per - 1) / per;                         // drop empty trailing splits
}

// out[M,N] = epilogue(A[M,K] . W[N,K]^T) for 1 <= M <= 64; A, W bf16 row-major (lda, ldw multiples of 8,
// 16-byte aligned bases), N even, `partial` = ps_gemm_smallm_splits(N, K) * M * N floats of scratch.
PS_API int ps_gemm_smallm(const void* a, int lda, const void* w, int ldw, int M, int N, int K, int epilogue, const void* residual,
                          int ld_res, void* out, int ldo, int out_f32, void* partial, void* status, cudaStream_t stream) {
    using namespace ps;
    if (M < 1 || M > 64 || N <= 0 || (N & 1) || K <= 0 || (K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)a % 16) ||
        ((uintptr_t)w % 16) || partial == nullptr)
        return (int)cudaErrorInvalidValue;
    if (epilogue == 2 && out_f32) return (int)cudaErrorInvalidValue;
    SmallMArgs g;
    g.M = M; g.N = N; g.K = K;
    g.nb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    g.x_box_rows = (M + 7) / 8 * 8;
    g.splits = ps_gemm_smallm_splits(N, K);
    const int iters = (K + kSmBK - 1) / kSmBK;
    g.iters_per_split = (iters + g.splits - 1) / g.splits;
    g.partial = (float*)partial; g.status = (uint32_t*)status; g.budget = g_ps_wait_budget_cycles;
    CUtensorMap map_w, map_x;
    int err = sm_map_2d(&map_w, w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, kSmBM);
    if (err) return err;
    err = sm_map_2d(&map_x, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint32_t)g.x_box_rows);
    if (err) return err;
    constexpr int STAGES = 4;
    const size_t smem = (size_t)STAGES * (kSmBM * kSmBK * 2 + 64 * kSmBK * 2) + 1024;       // 4 x 24 KB + alignment slack
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_smallm_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_smallm_kernel<STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        attr_set = true;
    }
    dim3 grid((N + kSmBM - 1) / kSmBM, g.splits);
    gemm_smallm_kernel<STAGES><<<grid, kSmThreads, smem, stream>>>(map_w, map_x, g);
    err = PS_LAUNCH_CHECK();
    if (err) return err;
    SmallMReduceArgs r;
    r.partial = g.partial; r.splits = g.splits; r.M = M; r.N = N; r.epilogue = epilogue;
    r.residual = (const __nv_bfloat16*)residual; r.ld_res = ld_res; r.out = out; r.ldo = ldo; r.out_f32 = out_f32;
    const long long n = (long long)M * (N >> 1);
    gemm_smallm_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(r);
    return PS_LAUNCH_CHECK();
}
