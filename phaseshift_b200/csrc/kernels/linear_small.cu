// Small-M linear launcher: fused prologue (RMSNorm / sigmoid gate), streaming GEMV over BF16 / NVFP4 /
// MXFP8 weights, fused epilogue (residual add / SwiGLU).  See gemv_core.cuh for the decomposition.
#include "gemv_core.cuh"

namespace ps {

template <int WF, int MT>
__global__ void __launch_bounds__(kGemvThreads, 2) linear_small_kernel(const LinearSmallArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    using XS = typename WTraits<WF>::XS;
    using DC = DotChunk<WF, MT>;
    constexpr int CH = WTraits<WF>::kChunk;
    constexpr int R = kRowsPerUnit;
    const int kpad = gemv_kpad<WF>(a.K);
    XS* xs = reinterpret_cast<XS*>(smem_raw);
    float* partial = reinterpret_cast<float*>(smem_raw + (size_t)kpad * MT * sizeof(XS));   // [kWavePairs][warps][R*MT]
    __shared__ float s_xscale_inv[MT], s_red[32];

    // Programmatic dependent launch: let the next kernel in the stream start its own weight prefetch
    // while this one runs; it blocks in cudaGridDependencySynchronize() until this grid has finished.
    cudaTriggerProgrammaticLaunchCompletion();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_pairs = (a.N + R - 1) / R;
    const int steps = GemvGeom::steps_for(a.K, CH);
    int pair_begin, pair_end;
    gemv_cta_pairs(n_pairs, gridDim.x, blockIdx.x, pair_begin, pair_end);

    // ---- first ring fill: weights only, independent of the previous kernel's output
    typename DC::Frag ring[kPrefetch][R];
    UnitWalker L;
    L.init(pair_begin, pair_end, steps, warp);
#pragma unroll
    for (int s = 0; s < kPrefetch; ++s) {
        int p, st;
        if (L.unit(p, st)) {
            const int k = (st * 32 + lane) * CH;
            if (k < a.K) {
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (p * R + r < a.N) DC::load(ring[s][r], a, p * R + r, k);
            }
        }
        L.next();
    }

    cudaGridDependencySynchronize();
    stage_rows<WF, MT>(a, xs, kpad, s_xscale_inv, s_red);
    for (int i = threadIdx.x; i < kWavePairs * kGemvWarps * R * MT; i += kGemvThreads) partial[i] = 0.f;
    __syncthreads();

    // ---- stream
    for (int wave_p0 = pair_begin; wave_p0 < pair_end; wave_p0 += kWavePairs) {
        const int wave_pairs = min(kWavePairs, pair_end - wave_p0);
        const int total = wave_pairs * steps;
        const int u0 = (total * warp) / kGemvWarps, u_end = (total * (warp + 1)) / kGemvWarps;
        float acc[R][MT];
        int cur_pair = -1;
        auto flush = [&]() {
            if (cur_pair < 0) return;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float v = warp_sum(acc[r][m]);
                    if (lane == 0) partial[((cur_pair - wave_p0) * kGemvWarps + warp) * (R * MT) + r * MT + m] = v;
                }
        };
        for (int base = u0; base < u_end; base += kPrefetch) {
#pragma unroll
            for (int s = 0; s < kPrefetch; ++s) {
                const int u = base + s;
                if (u < u_end) {
                    const int p = wave_p0 + u / steps, st = u % steps;
                    if (p != cur_pair) {
                        flush();
                        cur_pair = p;
#pragma unroll
                        for (int r = 0; r < R; ++r)
#pragma unroll
                            for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
                    }
                    const int k = (st * 32 + lane) * CH;
                    if (k < a.K) {
#pragma unroll
                        for (int r = 0; r < R; ++r)
                            if (p * R + r < a.N) DC::fma(ring[s][r], xs, kpad, k, acc[r]);
                    }
                }
                // refill this slot with the unit kPrefetch positions ahead in the padded stream
                int lp, lst;
                if (L.unit(lp, lst)) {
                    const int k = (lst * 32 + lane) * CH;
                    if (k < a.K) {
#pragma unroll
                        for (int r = 0; r < R; ++r)
                            if (lp * R + r < a.N) DC::load(ring[s][r], a, lp * R + r, k);
                    }
                }
                L.next();
            }
        }
        flush();
        __syncthreads();
        // ---- combine the warps' partial sums in warp order, apply the epilogue
        for (int i = threadIdx.x; i < wave_pairs * MT; i += kGemvThreads) {
            const int pl = i / MT, m = i % MT;
            float v[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) {
                    float* pp = &partial[(pl * kGemvWarps + w) * (R * MT) + r * MT + m];
                    s += *pp;
                    *pp = 0.f;
                }
                v[r] = s * (a.w_gscale * s_xscale_inv[m]);
            }
            if (m >= a.M) continue;
            const int n0 = (wave_p0 + pl) * R;
            if (a.epilogue == EPI_SWIGLU) {
                // rows (2j, 2j+1) hold (gate_j, up_j); both rounded to bf16 as separate projections would be
                if (n0 + 1 < a.N) {
                    const float g = bf16_to_f32(f32_to_bf16(v[0])), u = bf16_to_f32(f32_to_bf16(v[1]));
                    const float y = silu_f(g) * u;
                    if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + (n0 >> 1)] = y;
                    else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + (n0 >> 1)] = f32_to_bf16(y);
                }
                continue;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int n = n0 + r;
                if (n >= a.N) continue;
                float y = v[r];
                if (a.epilogue == EPI_RESIDUAL)   // y rounded to bf16 before the add, like projection-then-add
                    y = bf16_to_f32(f32_to_bf16(y)) + bf16_to_f32(a.residual[(size_t)m * a.ld_res + n]);
                if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n] = y;
                else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + n] = f32_to_bf16(y);
            }
        }
        __syncthreads();
    }
}

static int g_sm_count = 0;
static int g_pdl = -1;

template <int WF, int MT>
static int launch_small(const LinearSmallArgs& a, cudaStream_t stream) {
    const int kpad = gemv_kpad<WF>(a.K);
    const size_t smem = (size_t)kpad * MT * sizeof(typename WTraits<WF>::XS) +
                        sizeof(float) * kWavePairs * kGemvWarps * kRowsPerUnit * MT;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(linear_small_kernel<WF, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set = true;
    }
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        const char* e = getenv("PS_PDL");
        g_pdl = (e == nullptr || e[0] != '0') ? 1 : 0;
    }
    const int grid = gemv_grid(a.N, 2 * g_sm_count);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kGemvThreads); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, linear_small_kernel<WF, MT>, a);
}

template <int WF>
static int dispatch_m(const LinearSmallArgs& a, cudaStream_t stream) {
    if (a.M <= 1) return launch_small<WF, 1>(a, stream);
    if (a.M <= 2) return launch_small<WF, 2>(a, stream);
    if (a.M <= 4) return launch_small<WF, 4>(a, stream);
    if (a.M <= 8) return launch_small<WF, 8>(a, stream);
    return (int)cudaErrorInvalidValue;
}

}  // namespace ps

// y = epilogue( prologue(x) . W^T ), M <= 8.  Returns a cudaError_t value.
PS_API int ps_linear_small(int wfmt, const void* x, int M, int N, int K, int ldx, const void* w,
                           const void* w_scale, float w_gscale, int prologue, const void* norm_w, float eps,
                           const void* gate, int ld_gate, int epilogue, const void* residual, int ld_res,
                           void* out, int ldo, int out_f32, cudaStream_t stream) {
    using namespace ps;
    if (M < 1 || M > 8 || (K % 32) != 0 || (ldx % 8) != 0) return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && (N & 1)) return (int)cudaErrorInvalidValue;
    LinearSmallArgs a;
    a.x = (const __nv_bfloat16*)x; a.M = M; a.N = N; a.K = K; a.ldx = ldx;
    a.w = w; a.w_scale = (const uint8_t*)w_scale; a.w_gscale = w_gscale;
    a.prologue = prologue; a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps;
    a.gate = (const __nv_bfloat16*)gate; a.ld_gate = ld_gate;
    a.epilogue = epilogue; a.residual = (const __nv_bfloat16*)residual; a.ld_res = ld_res;
    a.out = out; a.ldo = ldo; a.out_f32 = out_f32;
    switch (wfmt) {
        case W_BF16: return dispatch_m<W_BF16>(a, stream);
        case W_NVFP4: return dispatch_m<W_NVFP4>(a, stream);
        case W_MXFP8: return dispatch_m<W_MXFP8>(a, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// Largest M x K the small-M kernel can stage at once for a format (callers split M above it).
PS_API int ps_linear_small_max_rows(int wfmt, int K) {
    using namespace ps;
    for (int mt = 8; mt >= 1; mt >>= 1) {
        size_t per = wfmt == W_BF16 ? (size_t)gemv_kpad<W_BF16>(K) * 4
                                    : (wfmt == W_NVFP4 ? (size_t)gemv_kpad<W_NVFP4>(K) * 2 : (size_t)gemv_kpad<W_MXFP8>(K) * 2);
        if (per * mt + sizeof(float) * kWavePairs * kGemvWarps * kRowsPerUnit * mt <= 200 * 1024) return mt;
    }
    return 0;
}
