// Small-M linear launcher: fused prologue (RMSNorm / sigmoid gate), GEMV over BF16 / NVFP4 / MXFP8
// weights, fused epilogue (residual add / SwiGLU).  See gemv_core.cuh for the contract.
#include "gemv_core.cuh"

namespace ps {

template <int WF, int MT>
__global__ void __launch_bounds__(kGemvThreads, 2) linear_small_kernel(const LinearSmallArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    using XS = typename WTraits<WF>::XS;
    XS* xs = reinterpret_cast<XS*>(smem_raw);
    __shared__ float s_inv_rms[MT], s_xscale[MT], s_xscale_inv[MT], s_red[32];

    row_stats<WF, MT>(a, s_inv_rms, s_xscale, s_xscale_inv, s_red);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kGemvRowsPerCta + warp * kGemvRowsPerWarp;
    float acc[kGemvRowsPerWarp][MT];
    gemv_accumulate<WF, MT>(a, xs, s_inv_rms, s_xscale, n0, acc);

    if (lane != 0) return;
    if (a.epilogue == EPI_SWIGLU) {
        // rows (2j, 2j+1) hold (gate_j, up_j); kGemvRowsPerWarp == 2 keeps a pair inside one warp.
        const int j = n0 >> 1;
        if (n0 + 1 < a.N) {
            for (int m = 0; m < MT && m < a.M; ++m) {
                const float sc = a.w_gscale * s_xscale_inv[m];
                // gate and up are rounded to bf16 first, as separate projections would store them
                const float g = bf16_to_f32(f32_to_bf16(acc[0][m] * sc));
                const float u = bf16_to_f32(f32_to_bf16(acc[1][m] * sc));
                const float v = silu_f(g) * u;
                if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + j] = v;
                else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + j] = f32_to_bf16(v);
            }
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < kGemvRowsPerWarp; ++r) {
        const int n = n0 + r;
        if (n >= a.N) continue;
        for (int m = 0; m < MT && m < a.M; ++m) {
            float v = acc[r][m] * (a.w_gscale * s_xscale_inv[m]);
            if (a.epilogue == EPI_RESIDUAL) {
                // y is rounded to bf16 before the add, matching projection-then-add in two steps
                v = bf16_to_f32(f32_to_bf16(v)) + bf16_to_f32(a.residual[(size_t)m * a.ld_res + n]);
            }
            if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + n] = f32_to_bf16(v);
        }
    }
}

template <int WF, int MT>
static int launch_small(const LinearSmallArgs& a, cudaStream_t stream) {
    const int kc = gemv_kchunk<WF, MT>(a.K);
    const size_t smem = (size_t)kc * MT * sizeof(typename WTraits<WF>::XS);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(linear_small_kernel<WF, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kGemvSmemBudget + 1024);
        attr_set = true;
    }
    const int grid = (a.N + kGemvRowsPerCta - 1) / kGemvRowsPerCta;
    linear_small_kernel<WF, MT><<<grid, kGemvThreads, smem, stream>>>(a);
    return PS_LAUNCH_CHECK();
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
