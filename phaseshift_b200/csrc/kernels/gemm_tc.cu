// Large-M (prefill) GEMM on the 5th-generation tensor cores: out[M,N] = epilogue(A[M,K] . W[N,K]^T).
//
// Blackwell-native structure, hand-written in PTX (ps_tcgen05.cuh):
//   * operands are fetched by TMA (`cp.async.bulk.tensor.2d`, 128-byte swizzle, no multicast) into a
//     kStages-deep shared-memory ring guarded by full/empty mbarriers;
//   * one elected thread issues `tcgen05.mma.cta_group::1.kind::f16` (128 x BN x 16 per instruction,
//     bf16 operands straight from shared memory through matrix descriptors), the fp32 accumulator
//     lives in tensor memory (128 lanes x BN columns);
//   * `tcgen05.commit` releases ring slots back to the producer and finally signals the epilogue;
//   * four epilogue warps read the accumulator with `tcgen05.ld` (each warp its own 32-lane quadrant),
//     apply the fused epilogue (residual add / SwiGLU on interleaved gate-up columns / f32 or bf16
//     store) and write to global memory.
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 = epilogue.
// Every mbarrier wait is bounded; a timeout sets PS_DEV_WAIT_TIMEOUT in the status word, the CTA
// stops issuing, frees its tensor memory and returns.
//
// The reference's counterpart is its WMMA bf16 family (src/phaseshift/models/qwen35/kernels/optimized/
// linear/bf16.hip:10-339) and the Prefill2D PSQ kernels (linear/psq4.hip:505-667); quantised weights
// are expanded to a bf16 scratch matrix first (dequant_tiled.cu), so one GEMM serves every format.
#include "ps_tcgen05.cuh"

namespace ps {

enum GemmEpilogue : int { GEPI_STORE = 0, GEPI_RESIDUAL = 1, GEPI_SWIGLU = 2 };

constexpr int kBM = 128, kBK = 64;
constexpr int kGemmThreads = 192;

struct GemmArgs {
    int M, N, K;
    int epilogue;
    const __nv_bfloat16* residual; int ld_res;
    void* out; int ldo; int out_f32;
    uint32_t* status;
    long long budget;    // clock-cycle budget of every mbarrier wait
    int a_box_rows;      // rows fetched per A tile (a multiple of 8, <= 128); the rest of the tile stays zero
};

// BN x kGemmStages x CTAs per SM: <256, 4, 1> / <128, 4, 1> for prefill-sized M; <32, 5, 2> for M <= 128 (batched decode
// on resident bf16 weights), where the problem is a weight stream: narrow N tiles give every SM a slice even
// when N is 5120, and two co-resident CTAs per SM keep ~40 KB of weights in flight without wave quantisation.
template <int BN, int kGemmStages, int kMinBlocks>
__global__ void __launch_bounds__(kGemmThreads, kMinBlocks)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const GemmArgs g) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int kABytes = kBM * kBK * 2, kBBytes = BN * kBK * 2;
    // 1024-byte alignment is required by the 128-byte swizzle atoms
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;
    unsigned char* sB = smem + kGemmStages * kABytes;
    __shared__ __align__(8) uint64_t full_bar[kGemmStages], empty_bar[kGemmStages], acc_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_abort, s_issued, s_consumed;      // stages handed to TMA / waited for by the MMA thread

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Rasterisation: the M tiles of a band of up to 16 vary fastest, so the CTAs that run together share
    // a few weight tiles (each read from HBM once and then served by L2) and the whole activation band.
    const int tiles_m = (g.M + kBM - 1) / kBM, tiles_n = (g.N + BN - 1) / BN;
    const int band = tiles_m < 16 ? tiles_m : 16;
    const int per_band = band * tiles_n;
    const int first_m = ((int)blockIdx.x / per_band) * band;
    const int gm = min(band, tiles_m - first_m);
    const int in_band = (int)blockIdx.x - (first_m / band) * per_band;
    const int tile_m = first_m + in_band % gm, tile_n = in_band / gm;
    const int k_iters = (g.K + kBK - 1) / kBK;
    const int a_bytes = g.a_box_rows * kBK * 2;            // bytes one TMA load of A delivers
    if (g.a_box_rows < kBM) {
        // few-row problems fetch only the rows that exist; the remaining rows of every A stage are zeroed once
        for (int i = threadIdx.x; i < kGemmStages * kABytes / 16; i += kGemmThreads) reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // make the zeros visible to the tensor core's async reads
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) { tc::mbar_init(&full_bar[s], 1); tc::mbar_init(&empty_bar[s], 1); }
        tc::mbar_init(&acc_bar, 1);
        tc::fence_barrier_init();
        s_abort = 0; s_issued = 0; s_consumed = 0;
        tc::tma_prefetch_desc(&map_a);
        tc::tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tc::tmem_alloc(&tmem_base_slot, BN);       // BN fp32 columns x 128 lanes
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_acc = tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < k_iters; ++it) {
                const int s = it % kGemmStages;
                const uint32_t ph = (uint32_t)(it / kGemmStages) & 1u;
                if (it >= kGemmStages && !tc::mbar_wait(&empty_bar[s], ph ^ 1u, g.budget)) { atomicExch(&s_abort, 1); break; }
                tc::mbar_expect_tx(&full_bar[s], a_bytes + kBBytes);
                tc::tma_load_2d(sA + s * kABytes, &map_a, it * kBK, tile_m * kBM, &full_bar[s]);
                tc::tma_load_2d(sB + s * kBBytes, &map_w, it * kBK, tile_n * BN, &full_bar[s]);
                s_issued = it + 1;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(kBM, BN);
            bool ok = true;
            for (int it = 0; it < k_iters && ok; ++it) {
                const int s = it % kGemmStages;
                const uint32_t ph = (uint32_t)(it / kGemmStages) & 1u;
                if (!tc::mbar_wait(&full_bar[s], ph, g.budget)) { atomicExch(&s_abort, 1); ok = false; break; }
                s_consumed = it + 1;
                tc::fence_after_sync();
                const uint32_t a_addr = tc::smem_u32(sA + s * kABytes), b_addr = tc::smem_u32(sB + s * kBBytes);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk) {
                    // advance 16 bf16 = 32 bytes inside the 128-byte swizzle row
                    const uint64_t adesc = tc::smem_desc_sw128(a_addr + kk * 32);
                    const uint64_t bdesc = tc::smem_desc_sw128(b_addr + kk * 32);
                    tc::mma_bf16_ss(tmem_acc, adesc, bdesc, idesc, (it > 0 || kk > 0) ? 1u : 0u);
                }
                tc::mma_commit(&empty_bar[s]);      // slot reusable once these MMAs have read it
            }
            tc::mma_commit(&acc_bar);               // accumulator complete (or whatever was issued)
        }
    } else {
        // ------------------------------------------------ epilogue: warps 2..5 -> TMEM lane quadrant (warp % 4)
        const int quad = warp & 3;
        const bool done = tc::mbar_wait(&acc_bar, 0, g.budget);
        tc::fence_after_sync();
        const int row = tile_m * kBM + quad * 32 + lane;
        if (done && s_abort == 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
                tc::tmem_ld_wait();
                const int col0 = tile_n * BN + c0;
                if (row < g.M) {
                    if (g.epilogue == GEPI_SWIGLU) {
                        // columns (2j, 2j+1) = (gate_j, up_j), each rounded to bf16 like a stored projection
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + (size_t)row * g.ldo + (col0 >> 1);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (col0 + 2 * j + 1 < g.N) {
                                const float gt = bf16_to_f32(f32_to_bf16(__uint_as_float(r[2 * j])));
                                const float up = bf16_to_f32(f32_to_bf16(__uint_as_float(r[2 * j + 1])));
                                o[j] = f32_to_bf16(silu_f(gt) * up);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const int col = col0 + j;
                            if (col + 1 < g.N) {
                                float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
                                if (g.epilogue == GEPI_RESIDUAL) {
                                    const float2 rs = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(
                                        g.residual + (size_t)row * g.ld_res + col));
                                    v0 = bf16_to_f32(f32_to_bf16(v0)) + rs.x;
                                    v1 = bf16_to_f32(f32_to_bf16(v1)) + rs.y;
                                }
                                if (g.out_f32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(g.out) + (size_t)row * g.ldo + col) = make_float2(v0, v1);
                                else *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(g.out) + (size_t)row * g.ldo + col) = f32x2_to_bf16x2_bits(v0, v1);
                            } else if (col < g.N) {
                                float v0 = __uint_as_float(r[j]);
                                if (g.epilogue == GEPI_RESIDUAL)
                                    v0 = bf16_to_f32(f32_to_bf16(v0)) + bf16_to_f32(g.residual[(size_t)row * g.ld_res + col]);
                                if (g.out_f32) reinterpret_cast<float*>(g.out)[(size_t)row * g.ldo + col] = v0;
                                else reinterpret_cast<__nv_bfloat16*>(g.out)[(size_t)row * g.ldo + col] = f32_to_bf16(v0);
                            }
                        }
                    }
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
        for (int c = s_consumed; c < s_issued; ++c) tc::mbar_wait(&full_bar[c % kGemmStages], (uint32_t)((c / kGemmStages) & 1), b);
    }
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_acc, BN);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D bf16 row-major [rows, cols] tensor map with a (box_rows x 64) box and 128-byte swizzle.
static int make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                       uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (enc == nullptr) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld_elems * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int BN, int kGemmStages, int kMinBlocks>
static int launch_gemm(const void* a, int lda, const void* w, int ldw, const GemmArgs& g, cudaStream_t stream) {
    CUtensorMap map_a, map_w;
    int err = make_map_2d(&map_a, a, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)lda, (uint32_t)g.a_box_rows);
    if (err) return err;
    err = make_map_2d(&map_w, w, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)ldw, BN);
    if (err) return err;
    const size_t smem = (size_t)kGemmStages * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN, kGemmStages, kMinBlocks>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN, kGemmStages, kMinBlocks>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        attr_set = true;
    }
    dim3 grid(((g.N + BN - 1) / BN) * ((g.M + kBM - 1) / kBM));
    gemm_bf16_tc_kernel<BN, kGemmStages, kMinBlocks><<<grid, kGemmThreads, smem, stream>>>(map_a, map_w, g);
    return PS_LAUNCH_CHECK();
}

}  // namespace ps

// out[M,N] = epilogue(A[M,K] . W[N,K]^T); A, W bf16 row-major (leading dimensions in elements, both
// multiples of 8 and base pointers 16-byte aligned, as TMA requires).
PS_API int ps_gemm_bf16_tc(const void* a, int lda, const void* w, int ldw, int M, int N, int K, int epilogue,
                           const void* residual, int ld_res, void* out, int ldo, int out_f32, void* status,
                           cudaStream_t stream) {
    using namespace ps;
    if (M <= 0 || N <= 0 || K <= 0 || (lda % 8) || (ldw % 8) || (K % 8) || ((uintptr_t)a % 16) || ((uintptr_t)w % 16))
        return (int)cudaErrorInvalidValue;
    if (epilogue == GEPI_SWIGLU && ((N & 1) || out_f32)) return (int)cudaErrorInvalidValue;
    GemmArgs g;
    g.M = M; g.N = N; g.K = K; g.epilogue = epilogue; g.residual = (const __nv_bfloat16*)residual; g.ld_res = ld_res;
    g.out = out; g.ldo = ldo; g.out_f32 = out_f32; g.status = (uint32_t*)status;
    g.budget = g_ps_wait_budget_cycles;
    g.a_box_rows = M >= kBM ? kBM : ((M + 7) / 8) * 8;
    if (M <= kBM && N >= 512) return launch_gemm<32, 5, 2>(a, lda, w, ldw, g, stream);
    if (N >= 256) return launch_gemm<256, 4, 1>(a, lda, w, ldw, g, stream);
    return launch_gemm<128, 4, 1>(a, lda, w, ldw, g, stream);
}
