// Small-M ("decode / verify") linear layer core: y[M,N] = prologue(x)[M,K] . W[N,K]^T.
//
// This is the memory-bound regime (M <= 8): every weight byte is read exactly once from
// HBM by exactly one warp, activations are staged once per CTA in shared memory, and all
// elementwise work around the projection (RMSNorm, sigmoid gate, residual add, SwiGLU)
// is folded into the prologue/epilogue so a transformer layer needs no standalone
// elementwise launches.  The per-row arithmetic does not depend on M, so a row computed
// in an M=1 launch and the same row computed inside an M=8 launch are bit-identical: this
// is the property the reference obtains with its ExactRows GEMM
// (src/phaseshift/models/qwen35/kernels/optimized/linear/bf16.hip:429-512) and that greedy
// speculative verification relies on.
//
// Weight formats (K contiguous, one row per output feature):
//   W_BF16  : bf16 [N,K]
//   W_NVFP4 : E2M1 nibbles [N,K/2] (byte j = q[2j] | q[2j+1] << 4), UE4M3 scale per 16
//             weights [N,K/16], one fp32 scale per tensor.  Replaces PSQ4
//             (src/.../linear/psq4.hip) on Blackwell.
//   W_MXFP8 : E4M3 bytes [N,K], UE8M0 scale per 32 weights [N,K/32].  Replaces PSQ8.
#pragma once

#include <cuda_fp4.h>

#include "ps_common.cuh"

namespace ps {

enum WeightFormat : int { W_BF16 = 0, W_NVFP4 = 1, W_MXFP8 = 2 };
enum LinearPrologue : int { PRO_NONE = 0, PRO_RMSNORM_ONEPLUS = 1, PRO_SIGMOID_GATE = 2 };
enum LinearEpilogue : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };

struct LinearSmallArgs {
    const __nv_bfloat16* x;   // [M, ldx]
    int M, N, K, ldx;
    const void* w;            // weight codes (format dependent)
    const uint8_t* w_scale;   // block scales (NVFP4 / MXFP8) or nullptr
    float w_gscale;           // per-tensor scale (NVFP4), 1 otherwise
    int prologue;
    const __nv_bfloat16* norm_w;  // [K] for PRO_RMSNORM_ONEPLUS
    float eps;
    const __nv_bfloat16* gate;    // PRO_SIGMOID_GATE: [M, ld_gate], x *= sigmoid(gate)
    int ld_gate;
    int epilogue;
    const __nv_bfloat16* residual;  // EPI_RESIDUAL: [M, ld_res]
    int ld_res;
    void* out;                // [M, ldo] bf16 or f32 ; EPI_SWIGLU writes N/2 features
    int ldo;
    int out_f32;
};

template <int WF> struct WTraits;
template <> struct WTraits<W_BF16>  { static constexpr int kChunk = 8;  using XS = float; };
template <> struct WTraits<W_NVFP4> { static constexpr int kChunk = 32; using XS = __half; };
template <> struct WTraits<W_MXFP8> { static constexpr int kChunk = 16; using XS = __half; };

// Largest |x| the staged fp16 activations may take so that an 8-term (NVFP4: |w|<=6) or
// 8-term (MXFP8: |w|<=448) half2 partial sum cannot overflow fp16.
template <int WF> __device__ __forceinline__ float stage_target_absmax() {
    return WF == W_NVFP4 ? 512.f : (WF == W_MXFP8 ? 8.f : 0.f);
}

// Stage prologue(x[m, k0:k0+kc]) for all m < M into shared memory (XS type), scaled by
// `xscale[m]` (a power of two; 1 for the fp32 path).
template <int WF, int MT>
__device__ __forceinline__ void stage_x(const LinearSmallArgs& a, typename WTraits<WF>::XS* xs,
                                        int k0, int kc, const float* inv_rms, const float* xscale) {
    using XS = typename WTraits<WF>::XS;
    for (int m = 0; m < MT; ++m) {
        const bool live = m < a.M;
        const __nv_bfloat16* xr = a.x + (size_t)m * a.ldx + k0;
        for (int k = threadIdx.x * 2; k < kc; k += blockDim.x * 2) {
            float v0 = 0.f, v1 = 0.f;
            if (live) {
                const float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + k));
                v0 = xv.x; v1 = xv.y;
                if (a.prologue == PRO_RMSNORM_ONEPLUS) {
                    const float2 wv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a.norm_w + k0 + k));
                    // y = bf16( x * rsqrt(mean(x^2)+eps) * (1 + w) ): rounded to bf16 like a standalone norm.
                    v0 = bf16_to_f32(f32_to_bf16(v0 * inv_rms[m] * (1.f + wv.x)));
                    v1 = bf16_to_f32(f32_to_bf16(v1 * inv_rms[m] * (1.f + wv.y)));
                } else if (a.prologue == PRO_SIGMOID_GATE) {
                    const float2 gv = bf16x2_bits_to_f32x2(
                        *reinterpret_cast<const uint32_t*>(a.gate + (size_t)m * a.ld_gate + k0 + k));
                    v0 = bf16_to_f32(f32_to_bf16(v0 * sigmoid_f(gv.x)));
                    v1 = bf16_to_f32(f32_to_bf16(v1 * sigmoid_f(gv.y)));
                }
                v0 *= xscale[m]; v1 *= xscale[m];
            }
            if constexpr (sizeof(XS) == 4) {
                *reinterpret_cast<float2*>(xs + (size_t)m * kc + k) = make_float2(v0, v1);
            } else {
                *reinterpret_cast<__half2*>(xs + (size_t)m * kc + k) = __floats2half2_rn(v0, v1);
            }
        }
    }
}

// Row statistics needed before staging: 1/rms for the RMSNorm prologue, and the power-of-two
// scale that maps the row's (post-prologue) absmax near `target` for the fp16 paths.
template <int WF, int MT>
__device__ __forceinline__ void row_stats(const LinearSmallArgs& a, float* inv_rms, float* xscale,
                                          float* xscale_inv, float* red) {
    const float target = stage_target_absmax<WF>();
    for (int m = 0; m < MT; ++m) {
        float ss = 0.f, amax = 0.f;
        if (m < a.M) {
            const __nv_bfloat16* xr = a.x + (size_t)m * a.ldx;
            if (a.prologue == PRO_RMSNORM_ONEPLUS) {
                for (int k = threadIdx.x * 2; k < a.K; k += blockDim.x * 2) {
                    const float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + k));
                    ss += xv.x * xv.x + xv.y * xv.y;
                }
                ss = block_sum(ss, red);
            }
            const float ir = (a.prologue == PRO_RMSNORM_ONEPLUS) ? rsqrtf(ss / (float)a.K + a.eps) : 1.f;
            if (threadIdx.x == 0) inv_rms[m] = ir;
            if (target > 0.f) {
                for (int k = threadIdx.x * 2; k < a.K; k += blockDim.x * 2) {
                    float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + k));
                    if (a.prologue == PRO_RMSNORM_ONEPLUS) {
                        const float2 wv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a.norm_w + k));
                        xv.x *= ir * (1.f + wv.x); xv.y *= ir * (1.f + wv.y);
                    }
                    // the sigmoid gate only shrinks |x|, so the ungated absmax is a valid bound
                    amax = fmaxf(amax, fmaxf(fabsf(xv.x), fabsf(xv.y)));
                }
                amax = block_max(amax, red);
            }
        }
        if (threadIdx.x == 0) {
            float s = 1.f;
            if (target > 0.f && amax > 0.f && amax < 3.0e38f) {
                int e; frexpf(target / amax, &e);   // target/amax = f * 2^e, f in [0.5,1)
                e = max(-60, min(60, e - 1));
                s = ldexpf(1.f, e);
            }
            xscale[m] = s;
            xscale_inv[m] = 1.f / s;
            if (m >= a.M) inv_rms[m] = 0.f;
        }
    }
    __syncthreads();
}

// One lane's contribution for one K-chunk position: `CH` consecutive weights of one output row
// against the staged activations of every batch row.
template <int WF, int MT> struct DotChunk;

template <int MT> struct DotChunk<W_BF16, MT> {
    struct Frag { uint4 w; };
    __device__ static __forceinline__ void load(Frag& f, const LinearSmallArgs& a, int n, int kabs) {
        f.w = __ldg(reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(a.w) + (size_t)n * a.K + kabs));
    }
    __device__ static __forceinline__ void fma(const Frag& f, const float* xs, int kc, int krel, float* acc) {
        const float2 w0 = bf16x2_bits_to_f32x2(f.w.x), w1 = bf16x2_bits_to_f32x2(f.w.y);
        const float2 w2 = bf16x2_bits_to_f32x2(f.w.z), w3 = bf16x2_bits_to_f32x2(f.w.w);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + (size_t)m * kc + krel);
            const float4 xb = *reinterpret_cast<const float4*>(xs + (size_t)m * kc + krel + 4);
            float s = acc[m];
            s = fmaf(w0.x, xa.x, s); s = fmaf(w0.y, xa.y, s);
            s = fmaf(w1.x, xa.z, s); s = fmaf(w1.y, xa.w, s);
            s = fmaf(w2.x, xb.x, s); s = fmaf(w2.y, xb.y, s);
            s = fmaf(w3.x, xb.z, s); s = fmaf(w3.y, xb.w, s);
            acc[m] = s;
        }
    }
};

__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
    __half2_raw r = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
    return *reinterpret_cast<__half2*>(&r);
}
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t two_bytes) {
    __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_bytes, __NV_E4M3);
    return *reinterpret_cast<__half2*>(&r);
}

template <int MT> struct DotChunk<W_NVFP4, MT> {
    struct Frag { uint4 w; uint32_t sc; };
    __device__ static __forceinline__ void load(Frag& f, const LinearSmallArgs& a, int n, int kabs) {
        f.w = __ldg(reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint8_t*>(a.w) + (size_t)n * (a.K >> 1) + (kabs >> 1)));
        f.sc = __ldg(reinterpret_cast<const uint16_t*>(a.w_scale + (size_t)n * (a.K >> 4) + (kabs >> 4)));
    }
    __device__ static __forceinline__ void fma(const Frag& f, const __half* xs, int kc, int krel, float* acc) {
        const float2 sc = __half22float2(e4m3x2_to_half2(f.sc));
        const uint32_t wq[4] = {f.w.x, f.w.y, f.w.z, f.w.w};
        __half2 wh[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) wh[j] = e2m1x2_to_half2((wq[j >> 2] >> ((j & 3) * 8)) & 0xffu);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * kc + krel);
            float s = acc[m];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const uint4 x0 = xp[b * 2], x1 = xp[b * 2 + 1];
                const uint32_t xr[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                __half2 p = __floats2half2_rn(0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    p = __hfma2(wh[b * 8 + j], *reinterpret_cast<const __half2*>(&xr[j]), p);
                const float2 pf = __half22float2(p);
                s = fmaf(pf.x + pf.y, b == 0 ? sc.x : sc.y, s);
            }
            acc[m] = s;
        }
    }
};

template <int MT> struct DotChunk<W_MXFP8, MT> {
    struct Frag { uint4 w; uint32_t sc; };
    __device__ static __forceinline__ void load(Frag& f, const LinearSmallArgs& a, int n, int kabs) {
        f.w = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.w) + (size_t)n * a.K + kabs));
        f.sc = __ldg(a.w_scale + (size_t)n * (a.K >> 5) + (kabs >> 5));
    }
    __device__ static __forceinline__ void fma(const Frag& f, const __half* xs, int kc, int krel, float* acc) {
        const float sc = __uint_as_float(f.sc << 23);   // UE8M0: 2^(e-127); e=0 decodes to 0 (unused)
        const uint32_t wq[4] = {f.w.x, f.w.y, f.w.z, f.w.w};
        __half2 wh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) wh[j] = e4m3x2_to_half2((wq[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * kc + krel);
            const uint4 x0 = xp[0], x1 = xp[1];
            const uint32_t xr[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            __half2 p = __floats2half2_rn(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) p = __hfma2(wh[j], *reinterpret_cast<const __half2*>(&xr[j]), p);
            const float2 pf = __half22float2(p);
            acc[m] = fmaf(pf.x + pf.y, sc, acc[m]);
        }
    }
};

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvRowsPerWarp = 2;
constexpr int kGemvRowsPerCta = kGemvWarps * kGemvRowsPerWarp;
constexpr int kGemvSmemBudget = 96 * 1024;

// K extent staged at once: a multiple of 32 lanes x chunk, at most the budget allows.
template <int WF, int MT>
__host__ __device__ inline int gemv_kchunk(int K) {
    constexpr int unit = 32 * WTraits<WF>::kChunk;
    const int esz = (int)sizeof(typename WTraits<WF>::XS);
    int kc = (kGemvSmemBudget / (MT * esz)) / unit * unit;
    const int kpad = (K + unit - 1) / unit * unit;
    return kc < kpad ? kc : kpad;
}

// Accumulate acc[r][m] = sum_k W[n0 + r][k] * xstaged[m][k] for this warp's rows.  The reduction
// order over k is a fixed function of (lane, K) only.
template <int WF, int MT, typename Args>
__device__ __forceinline__ void gemv_accumulate(const Args& a, typename WTraits<WF>::XS* xs,
                                                const float* inv_rms, const float* xscale,
                                                int n0, float (&acc)[kGemvRowsPerWarp][MT]) {
    constexpr int CH = WTraits<WF>::kChunk;
    using DC = DotChunk<WF, MT>;
    const int lane = threadIdx.x & 31;
    const int kc_full = gemv_kchunk<WF, MT>(a.K);
#pragma unroll
    for (int r = 0; r < kGemvRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

    for (int k0 = 0; k0 < a.K; k0 += kc_full) {
        const int kc = min(kc_full, a.K - k0);
        if (k0 > 0) __syncthreads();
        stage_x<WF, MT>(a, xs, k0, kc, inv_rms, xscale);
        __syncthreads();
        const int steps = (kc + 32 * CH - 1) / (32 * CH);
        constexpr int U = 4;
        for (int s0 = 0; s0 < steps; s0 += U) {
            typename DC::Frag fr[U][kGemvRowsPerWarp];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int krel = ((s0 + u) * 32 + lane) * CH;
#pragma unroll
                for (int r = 0; r < kGemvRowsPerWarp; ++r)
                    if (krel < kc && n0 + r < a.N) DC::load(fr[u][r], a, n0 + r, k0 + krel);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int krel = ((s0 + u) * 32 + lane) * CH;
                if (krel < kc) {
#pragma unroll
                    for (int r = 0; r < kGemvRowsPerWarp; ++r)
                        if (n0 + r < a.N) DC::fma(fr[u][r], xs, kc, krel, acc[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kGemvRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = warp_sum(acc[r][m]);
}

}  // namespace ps
