// Small-M ("decode / verify") linear layer core: y[M,N] = prologue(x)[M,K] . W[N,K]^T.
//
// This is the memory-bound regime (M <= 8): every weight byte is read exactly once from HBM,
// activations are staged once per CTA in shared memory, and all elementwise work around the
// projection (RMSNorm, sigmoid gate, residual add, SwiGLU) is folded into the prologue/epilogue so a
// transformer layer needs no standalone elementwise launches.
//
// Work decomposition (persistent CTAs, <= 2 per SM):
//   * output rows are taken in pairs; CTA c owns a contiguous range of pairs, processed in waves of
//     at most kWavePairs pairs;
//   * inside a wave the (pair, k-step) units are split into 8 contiguous, equal ranges, one per
//     warp, so every warp streams the same number of bytes whatever N and K are (a 48-row projection
//     and a 152k-row lm_head both keep all warps busy);
//   * each lane keeps kPrefetch 16-byte weight loads in flight at all times: a register ring is
//     refilled with the unit kPrefetch ahead right after a slot is consumed, across pair and wave
//     boundaries, and the first ring fill is issued before the activations are even staged;
//   * a warp's partial sums for a pair go to shared memory and are combined in warp order.
// The assignment of units to warps and the combination order are functions of (N, K, gridDim) only,
// never of M, so a row computed in an M=1 launch and the same row inside an M=8 launch are
// bit-identical: the property the reference obtains with its ExactRows GEMM
// (src/phaseshift/models/qwen35/kernels/optimized/linear/bf16.hip:429-512) and that greedy
// speculative verification relies on.
//
// Weight formats (K contiguous, one row per output feature):
//   W_BF16  : bf16 [N,K]
//   W_NVFP4 : E2M1 nibbles [N,K/2] (byte j = q[2j] | q[2j+1] << 4), UE4M3 scale per 16 weights
//             [N,K/16], one fp32 scale per tensor.  Replaces PSQ4 (src/.../linear/psq4.hip).
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

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kRowsPerUnit = 2;      // a unit = one k-step of a pair of output rows
constexpr int kWavePairs = 32;
constexpr int kPrefetch = 4;

// Largest |x| the staged fp16 activations may take so that an 8-term half2 partial sum (|w| <= 6 for
// NVFP4, <= 448 for MXFP8) cannot overflow fp16.
template <int WF> __device__ __forceinline__ float stage_target_absmax() {
    return WF == W_NVFP4 ? 512.f : (WF == W_MXFP8 ? 8.f : 0.f);
}

// Row statistics + staging of prologue(x) into shared memory (XS type), one pass over x per row:
// sum of squares (RMSNorm) and max |x (1+w)| (fp16 range scaling; the sigmoid gate only shrinks |x|).
template <int WF, int MT>
__device__ __forceinline__ void stage_rows(const LinearSmallArgs& a, typename WTraits<WF>::XS* xs, int kpad,
                                           float* xscale_inv, float* red) {
    using XS = typename WTraits<WF>::XS;
    const float target = stage_target_absmax<WF>();
    const bool norm = a.prologue == PRO_RMSNORM_ONEPLUS;
    for (int m = 0; m < MT; ++m) {
        const bool live = m < a.M;
        const __nv_bfloat16* xr = a.x + (size_t)m * a.ldx;
        float ss = 0.f, amax = 0.f;
        if (live && (norm || target > 0.f)) {
            for (int k = threadIdx.x * 2; k < a.K; k += kGemvThreads * 2) {
                float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + k));
                ss += xv.x * xv.x + xv.y * xv.y;
                if (norm) {
                    const float2 wv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a.norm_w + k));
                    xv.x *= 1.f + wv.x; xv.y *= 1.f + wv.y;
                }
                amax = fmaxf(amax, fmaxf(fabsf(xv.x), fabsf(xv.y)));
            }
            ss = block_sum(ss, red);
            amax = block_max(amax, red);
        }
        const float ir = norm ? rsqrtf(ss / (float)a.K + a.eps) : 1.f;
        float s = 1.f;
        if (target > 0.f) {
            const float am = amax * ir;
            if (am > 0.f && am < 3.0e38f) {
                int e; frexpf(target / am, &e);    // target/am = f * 2^e with f in [0.5, 1)
                s = ldexpf(1.f, max(-60, min(60, e - 1)));
            }
        }
        if (threadIdx.x == 0) xscale_inv[m] = 1.f / s;
        for (int k = threadIdx.x * 2; k < kpad; k += kGemvThreads * 2) {
            float v0 = 0.f, v1 = 0.f;
            if (live && k < a.K) {
                const float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + k));
                v0 = xv.x; v1 = xv.y;
                if (norm) {
                    const float2 wv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a.norm_w + k));
                    // rounded to bf16 like a standalone norm kernel would store it
                    v0 = bf16_to_f32(f32_to_bf16(v0 * ir * (1.f + wv.x)));
                    v1 = bf16_to_f32(f32_to_bf16(v1 * ir * (1.f + wv.y)));
                } else if (a.prologue == PRO_SIGMOID_GATE) {
                    const float2 gv = bf16x2_bits_to_f32x2(
                        *reinterpret_cast<const uint32_t*>(a.gate + (size_t)m * a.ld_gate + k));
                    v0 = bf16_to_f32(f32_to_bf16(v0 * sigmoid_f(gv.x)));
                    v1 = bf16_to_f32(f32_to_bf16(v1 * sigmoid_f(gv.y)));
                }
                v0 *= s; v1 *= s;
            }
            if constexpr (sizeof(XS) == 4) *reinterpret_cast<float2*>(xs + (size_t)m * kpad + k) = make_float2(v0, v1);
            else *reinterpret_cast<__half2*>(xs + (size_t)m * kpad + k) = __floats2half2_rn(v0, v1);
        }
    }
}

__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
    __half2_raw r = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
    return *reinterpret_cast<__half2*>(&r);
}
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t two_bytes) {
    __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_bytes, __NV_E4M3);
    return *reinterpret_cast<__half2*>(&r);
}

// One lane's share of a unit: kChunk consecutive weights of one output row against the staged
// activations of every batch row.
template <int WF, int MT> struct DotChunk;

template <int MT> struct DotChunk<W_BF16, MT> {
    struct Frag { uint4 w; };
    __device__ static __forceinline__ void load(Frag& f, const LinearSmallArgs& a, int n, int k) {
        f.w = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.w) + (size_t)n * a.K + k));
    }
    __device__ static __forceinline__ void fma(const Frag& f, const float* xs, int kpad, int k, float* acc) {
        const float2 w0 = bf16x2_bits_to_f32x2(f.w.x), w1 = bf16x2_bits_to_f32x2(f.w.y);
        const float2 w2 = bf16x2_bits_to_f32x2(f.w.z), w3 = bf16x2_bits_to_f32x2(f.w.w);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + (size_t)m * kpad + k);
            const float4 xb = *reinterpret_cast<const float4*>(xs + (size_t)m * kpad + k + 4);
            float s = acc[m];
            s = fmaf(w0.x, xa.x, s); s = fmaf(w0.y, xa.y, s);
            s = fmaf(w1.x, xa.z, s); s = fmaf(w1.y, xa.w, s);
            s = fmaf(w2.x, xb.x, s); s = fmaf(w2.y, xb.y, s);
            s = fmaf(w3.x, xb.z, s); s = fmaf(w3.y, xb.w, s);
            acc[m] = s;
        }
    }
};

template <int MT> struct DotChunk<W_NVFP4, MT> {
    struct Frag { uint4 w; uint32_t sc; };
    __device__ static __forceinline__ void load(Frag& f, const LinearSmallArgs& a, int n, int k) {
        f.w = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.w) + (size_t)n * (a.K >> 1) + (k >> 1)));
        f.sc = __ldcs(reinterpret_cast<const uint16_t*>(a.w_scale + (size_t)n * (a.K >> 4) + (k >> 4)));
    }
    __device__ static __forceinline__ void fma(const Frag& f, const __half* xs, int kpad, int k, float* acc) {
        const float2 sc = __half22float2(e4m3x2_to_half2(f.sc));
        const uint32_t wq[4] = {f.w.x, f.w.y, f.w.z, f.w.w};
        __half2 wh[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) wh[j] = e2m1x2_to_half2((wq[j >> 2] >> ((j & 3) * 8)) & 0xffu);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * kpad + k);
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
    __device__ static __forceinline__ void load(Frag& f, const LinearSmallArgs& a, int n, int k) {
        f.w = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.w) + (size_t)n * a.K + k));
        f.sc = __ldcs(a.w_scale + (size_t)n * (a.K >> 5) + (k >> 5));
    }
    __device__ static __forceinline__ void fma(const Frag& f, const __half* xs, int kpad, int k, float* acc) {
        const float sc = __uint_as_float(f.sc << 23);   // UE8M0: 2^(e-127)
        const uint32_t wq[4] = {f.w.x, f.w.y, f.w.z, f.w.w};
        __half2 wh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) wh[j] = e4m3x2_to_half2((wq[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * kpad + k);
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

// Geometry shared by host and device: which pairs a CTA owns.
struct GemvGeom {
    int n_pairs, steps, kpad;
    __host__ __device__ static int steps_for(int K, int chunk) { return (K + 32 * chunk - 1) / (32 * chunk); }
};
__host__ __device__ inline int gemv_grid(int N, int max_ctas) {
    const int n_pairs = (N + kRowsPerUnit - 1) / kRowsPerUnit;
    return n_pairs < max_ctas ? n_pairs : max_ctas;
}
template <int WF>
__host__ __device__ inline int gemv_kpad(int K) {
    constexpr int unit = 32 * WTraits<WF>::kChunk;
    return (K + unit - 1) / unit * unit;
}

// Walks one warp's unit stream in "padded" positions: the CTA's pairs are processed in waves of at
// most kWavePairs pairs; inside a wave the (pair, k-step) units are cut into kGemvWarps contiguous
// slices, and every slice is padded with null units to a multiple of kPrefetch so that stream
// position q always lives in ring slot q % kPrefetch (static register indexing).
struct UnitWalker {
    int pair_end, steps, warp;
    int wave_pair0, wave_pairs;   // current wave (wave_pairs <= 0: stream exhausted)
    int u0, u_end, q, q_end;      // slice [u0, u_end) of the wave, padded position q in [0, q_end)
    __device__ __forceinline__ void set_wave(int p0) {
        wave_pair0 = p0;
        wave_pairs = min(kWavePairs, pair_end - p0);
        q = 0;
        if (wave_pairs <= 0) { u0 = u_end = q_end = 0; return; }
        const int total = wave_pairs * steps;
        u0 = (total * warp) / kGemvWarps;
        u_end = (total * (warp + 1)) / kGemvWarps;
        q_end = (u_end - u0 + kPrefetch - 1) / kPrefetch * kPrefetch;
    }
    __device__ __forceinline__ void init(int pair_begin, int pair_end_, int steps_, int warp_) {
        pair_end = pair_end_; steps = steps_; warp = warp_;
        set_wave(pair_begin);
        while (wave_pairs > 0 && q >= q_end) set_wave(wave_pair0 + kWavePairs);
    }
    __device__ __forceinline__ bool exhausted() const { return wave_pairs <= 0; }
    // true when the current padded position is a real unit; then (pair, step) identify it
    __device__ __forceinline__ bool unit(int& pair, int& step) const {
        const int u = u0 + q;
        if (wave_pairs <= 0 || u >= u_end) return false;
        pair = wave_pair0 + u / steps; step = u % steps;
        return true;
    }
    __device__ __forceinline__ void next() {
        if (wave_pairs <= 0) return;
        ++q;
        while (wave_pairs > 0 && q >= q_end) set_wave(wave_pair0 + kWavePairs);
    }
};

// CTA c of `grid` owns pairs [begin, end): an even split with the remainder spread over the first CTAs.
__host__ __device__ inline void gemv_cta_pairs(int n_pairs, int grid, int c, int& begin, int& end) {
    const int base = n_pairs / grid, rem = n_pairs % grid;
    begin = c * base + (c < rem ? c : rem);
    end = begin + base + (c < rem ? 1 : 0);
}

}  // namespace ps
