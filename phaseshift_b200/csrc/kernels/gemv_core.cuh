// Small-M ("decode / verify") linear layer core: y[M,N] = prologue(x)[M,K] . W[N,K]^T.
//
// This is the memory-bound regime (M <= 8): every weight byte is read exactly once from HBM,
// activations are staged once per CTA in shared memory, and all elementwise work around the
// projection (RMSNorm, sigmoid gate, residual add, SwiGLU) is folded into the prologue/epilogue so a
// transformer layer needs no standalone elementwise launches.
//
// Weight storage ("tiled" layout, produced once at load time from the canonical row-major payload;
// the counterpart of the reference's mandatory native preshuffle,
// docs/developer/psq_canonical_soa_payload.md:674-708): output rows are grouped in quads, K in
// k-steps of 32 lanes x 16 bytes, and the bytes one warp consumes together are contiguous:
//     block(quad q, step s) at byte offset (q * steps + s) * kBlockBytes
//       [4 rows x 512 B of codes][4 rows x kScaleRow B of block scales]
// so a unit is ONE contiguous bulk copy and consecutive units of a warp form one sequential stream
// (DRAM sees long bursts instead of 512-byte fragments 10 KB apart).  N is padded to a multiple of 4
// and K to a whole k-step with zeros.
//   W_BF16  : 256 weights per row-step, no scales, 2048 B blocks
//   W_NVFP4 : 1024 E2M1 weights per row-step (byte j = q[2j] | q[2j+1] << 4), 64 UE4M3 scales per
//             row-step (one per 16 weights), 2304 B blocks, plus one fp32 scale per tensor.
//             Replaces PSQ4 (src/phaseshift/models/qwen35/kernels/optimized/linear/psq4.hip).
//   W_MXFP8 : 512 E4M3 weights per row-step, 16 UE8M0 scales (one per 32), 2112 B blocks.  Replaces PSQ8.
//
// Arithmetic: the assignment of (quad, k-step) units to warps and the order in which partial sums
// are combined are functions of (N, K, grid) only, never of M, so a row computed in an M=1 launch
// and the same row inside an M=4 launch are bit-identical: the property the reference obtains with
// its ExactRows GEMM (linear/bf16.hip:429-512) and that greedy speculative verification relies on.
#pragma once

#include "ps_common.cuh"

namespace ps {

enum WeightFormat : int { W_BF16 = 0, W_NVFP4 = 1, W_MXFP8 = 2 };
enum LinearPrologue : int { PRO_NONE = 0, PRO_RMSNORM_ONEPLUS = 1, PRO_SIGMOID_GATE = 2 };
enum LinearEpilogue : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };

constexpr int kTpMaxRanks = 8;
// Tensor-parallel combine fused into a row-parallel projection's epilogue (one-shot all-reduce over
// NVLink peer memory).  Every rank runs the same kernel with the same grid, so CTA c owns the same
// output rows everywhere: it pushes its fp32 partial sums into every rank's receive buffer with plain
// peer stores, raises a per-(CTA, source rank) flag with a system-scope release, waits (bounded) for
// the same CTA of every peer, then adds the partials in rank order 0..size-1 -- the identical order on
// every rank, so all ranks hold bit-identical results -- plus the residual.
// The reference combines with a separate leader-reduce + broadcast per projection and a host
// rendezvous (src/phaseshift/runtime/tp/hip_peer_tp_transport.hip:314-369, tp_barrier_group.cpp:74-119).
struct TpCombine {
    int size, rank;                       // size <= 1: disabled
    float* recv[kTpMaxRanks];             // rank r's receive buffer: [2 parities][size][max_rows][n_pad] f32
    uint32_t* flags[kTpMaxRanks];         // rank r's flags: [grid][size]
    uint32_t* counter;                    // local, [grid]: collectives this CTA has taken part in
    int max_rows, n_pad;
};

struct LinearSmallArgs {
    const __nv_bfloat16* x;   // [M, ldx]
    int M, N, K, ldx;         // K = logical reduction length (multiple of 32)
    const uint8_t* w;         // tiled weight blocks
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
    __nv_bfloat16* xn_out;    // optional [M, K]: the prologue's output row(s), written by CTA 0
    TpCombine tp;
    // Optional fused greedy sampling (the lm_head of a decode step): every CTA folds the rows it produced into a running
    // (value, index) best per batch row, the last CTA to finish writes the winners' indices and re-arms the state.
    unsigned long long* amax_best;   // [8] packed keys, zero between launches
    unsigned int* amax_ctl;          // [0] CTAs done, [1] a non-finite value was seen
    int* amax_tokens;                // [M] winners (-1 when a non-finite value was seen)
};

// Packed arg-max key: the value's bits made monotonic, then the complement of the index, so that an unsigned 64-bit maximum
// picks the larger value and, between equal values, the lower index (the sampling kernel's rule).
__device__ __forceinline__ unsigned long long amax_key(float v, int n) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)n);
}

constexpr int kQuadRows = 4;

template <int WF> struct WTraits;
template <> struct WTraits<W_BF16> {
    static constexpr int kChunk = 8, kScaleRow = 0, kBlockBytes = 2048;
    using XS = float;
};
template <> struct WTraits<W_NVFP4> {
    static constexpr int kChunk = 32, kScaleRow = 64, kBlockBytes = 2048 + 4 * 64;
    using XS = __half;
};
template <> struct WTraits<W_MXFP8> {
    static constexpr int kChunk = 16, kScaleRow = 16, kBlockBytes = 2048 + 4 * 16;
    using XS = __half;
};

template <int WF> __host__ __device__ constexpr int step_k() { return 32 * WTraits<WF>::kChunk; }
template <int WF> __host__ __device__ inline int gemv_steps(int K) { return (K + step_k<WF>() - 1) / step_k<WF>(); }
template <int WF> __host__ __device__ inline int gemv_kpad(int K) { return gemv_steps<WF>(K) * step_k<WF>(); }

// CTA c of `grid` owns items [begin, end): an even split with the remainder spread over the first CTAs.
__host__ __device__ inline void cta_range(int n_items, int grid, int c, int& begin, int& end) {
    const int base = n_items / grid, rem = n_items % grid;
    begin = c * base + (c < rem ? c : rem);
    end = begin + base + (c < rem ? 1 : 0);
}

// Largest |x| the staged fp16 activations may take so that an 8-term half2 partial sum (|w| <= 6 for
// NVFP4, <= 448 for MXFP8) cannot overflow fp16.
template <int WF> __device__ __forceinline__ float stage_target_absmax() {
    return WF == W_NVFP4 ? 512.f : (WF == W_MXFP8 ? 8.f : 0.f);
}

// Position of activation k inside the staged row.  A lane's kChunk activations of one k-step are
// several 16-byte groups; group q of lane l sits at 16-byte slot q * 32 + l of the step, so that the
// warp's q-th vector load touches 32 consecutive 16-byte slots (no shared-memory bank conflicts)
// instead of slots kChunk * sizeof(XS) bytes apart.
template <int WF> __device__ __forceinline__ int xpos(int k) {
    using XS = typename WTraits<WF>::XS;
    constexpr int EPG = 16 / (int)sizeof(XS);                       // elements per 16-byte group
    constexpr int GPL = WTraits<WF>::kChunk / EPG;                  // groups per lane
    constexpr int SK = 32 * WTraits<WF>::kChunk;                    // elements per k-step
    const int r = k % SK, g = r / EPG;
    return (k - r) + ((g % GPL) * 32 + g / GPL) * EPG + (r % EPG);
}

// Row statistics + staging of prologue(x) into shared memory (XS type), zero-padded to kpad.
// Pass 1 reads x from global once, parks the raw bf16 bits in the staging buffer and accumulates the
// sum of squares (RMSNorm) and max |x (1+w)| (fp16 range scaling; the sigmoid gate only shrinks |x|);
// pass 2 rewrites the buffer in place in its final form, so only one global round trip sits on the
// kernel's critical path.  With `xn_out` set, CTA 0 also stores the normalised row (bf16) to global
// for a consumer that needs it again (the GDN kernel's in-kernel b/a projections).
template <int WF, int MT, int THREADS>
__device__ __forceinline__ void stage_rows_generic(const LinearSmallArgs& a, typename WTraits<WF>::XS* xs, int kpad,
                                                float* xscale_inv, float* red) {
    using XS = typename WTraits<WF>::XS;
    const float target = stage_target_absmax<WF>();
    const bool norm = a.prologue == PRO_RMSNORM_ONEPLUS;
    for (int m = 0; m < MT; ++m) {
        const bool live = m < a.M;
        const __nv_bfloat16* xr = a.x + (size_t)m * a.ldx;
        XS* xrow = xs + (size_t)m * kpad;
        float ss = 0.f, amax = 0.f;
        for (int k = threadIdx.x * 2; k < kpad; k += THREADS * 2) {
            uint32_t bits = 0u;
            if (live && k < a.K) {
                bits = *reinterpret_cast<const uint32_t*>(xr + k);
                float2 xv = bf16x2_bits_to_f32x2(bits);
                ss += xv.x * xv.x + xv.y * xv.y;
                if (norm) {
                    const float2 wv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a.norm_w + k));
                    xv.x *= 1.f + wv.x; xv.y *= 1.f + wv.y;
                }
                amax = fmaxf(amax, fmaxf(fabsf(xv.x), fabsf(xv.y)));
            }
            const int kp = xpos<WF>(k);
            if constexpr (sizeof(XS) == 4) xrow[kp] = __uint_as_float(bits);           // raw bits parked in place
            else *reinterpret_cast<uint32_t*>(xrow + kp) = bits;
        }
        if (norm || target > 0.f) block_sum_max(ss, amax, red);
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
        for (int k = threadIdx.x * 2; k < kpad; k += THREADS * 2) {
            const int kp = xpos<WF>(k);
            uint32_t bits;
            if constexpr (sizeof(XS) == 4) bits = __float_as_uint(xrow[kp]);
            else bits = *reinterpret_cast<const uint32_t*>(xrow + kp);
            float2 xv = bf16x2_bits_to_f32x2(bits);
            float v0 = xv.x, v1 = xv.y;
            if (live && k < a.K) {
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
                if (a.xn_out != nullptr && blockIdx.x == 0)
                    *reinterpret_cast<uint32_t*>(a.xn_out + (size_t)m * a.K + k) = f32x2_to_bf16x2_bits(v0, v1);
            }
            v0 *= s; v1 *= s;
            if constexpr (sizeof(XS) == 4) *reinterpret_cast<float2*>(xrow + kp) = make_float2(v0, v1);
            else *reinterpret_cast<__half2*>(xrow + kp) = __floats2half2_rn(v0, v1);
        }
    }
}

// Fast path of stage_rows: every thread keeps its share of the row (up to kStageVec 16-byte vectors of
// eight activations) in registers between the statistics pass and the final write, so the row costs a
// single global round trip, no shared-memory parking and no second read of the norm weights.
constexpr int kStageVec = 6;

struct StageW { uint4 v[kStageVec]; };

// The norm weights do not depend on the producer grid: load them before waiting for it.
template <int THREADS>
__device__ __forceinline__ void stage_load_norm_w(const LinearSmallArgs& a, StageW& w) {
    const bool ok = a.prologue == PRO_RMSNORM_ONEPLUS && (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0;
    const int kvec = a.K >> 3;
#pragma unroll
    for (int j = 0; j < kStageVec; ++j) {
        const int idx = threadIdx.x + j * THREADS;
        w.v[j] = (ok && idx < kvec) ? __ldg(reinterpret_cast<const uint4*>(a.norm_w) + idx) : make_uint4(0, 0, 0, 0);
    }
}

template <int WF, int MT, int THREADS>
__device__ __forceinline__ void stage_rows(const LinearSmallArgs& a, typename WTraits<WF>::XS* xs, int kpad,
                                           float* xscale_inv, float* red, const StageW& sw) {
    using XS = typename WTraits<WF>::XS;
    const int nvec = kpad >> 3;
    const bool norm = a.prologue == PRO_RMSNORM_ONEPLUS, gated = a.prologue == PRO_SIGMOID_GATE;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) &&
                         (!norm || (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0) &&
                         (!gated || ((reinterpret_cast<uintptr_t>(a.gate) & 15) == 0 && (a.ld_gate & 7) == 0)) &&
                         (a.xn_out == nullptr || (reinterpret_cast<uintptr_t>(a.xn_out) & 15) == 0);
    if (nvec > kStageVec * THREADS || !aligned) { stage_rows_generic<WF, MT, THREADS>(a, xs, kpad, xscale_inv, red); return; }
    const float target = stage_target_absmax<WF>();
    const int kvec = a.K >> 3;                      // K is a multiple of 32
    const uint4 (&wv)[kStageVec] = sw.v;
    for (int m = 0; m < MT; ++m) {
        const bool live = m < a.M;
        const uint4* xr = reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx);
        XS* xrow = xs + (size_t)m * kpad;
        uint4 xv[kStageVec], gv[kStageVec];
#pragma unroll
        for (int j = 0; j < kStageVec; ++j) {
            const int idx = threadIdx.x + j * THREADS;
            const bool in = live && idx < kvec;
            xv[j] = in ? xr[idx] : make_uint4(0, 0, 0, 0);
            gv[j] = (gated && in) ? *(reinterpret_cast<const uint4*>(a.gate + (size_t)m * a.ld_gate) + idx) : make_uint4(0, 0, 0, 0);
        }
        float ss = 0.f, amax = 0.f;
#pragma unroll
        for (int j = 0; j < kStageVec; ++j) {
            const uint32_t xw[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
            const uint32_t ww[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 v = bf16x2_bits_to_f32x2(xw[e]);
                ss += v.x * v.x + v.y * v.y;
                if (norm) { const float2 w = bf16x2_bits_to_f32x2(ww[e]); v.x *= 1.f + w.x; v.y *= 1.f + w.y; }
                amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
            }
        }
        if (norm || target > 0.f) block_sum_max(ss, amax, red);
        const float ir = norm ? rsqrtf(ss / (float)a.K + a.eps) : 1.f;
        float s = 1.f;
        if (target > 0.f) {
            const float am = amax * ir;
            if (am > 0.f && am < 3.0e38f) {
                // target/am = f * 2^e with f in [0.5, 1): s = 2^(e-1), clamped
                const int e = (int)((__float_as_uint(target / am) >> 23) & 0xffu) - 126;
                s = __uint_as_float((uint32_t)(max(-60, min(60, e - 1)) + 127) << 23);
            }
        }
        if (threadIdx.x == 0) xscale_inv[m] = 1.f / s;
#pragma unroll
        for (int j = 0; j < kStageVec; ++j) {
            const int idx = threadIdx.x + j * THREADS;
            const uint32_t xw[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
            const uint32_t ww[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
            const uint32_t gw[4] = {gv[j].x, gv[j].y, gv[j].z, gv[j].w};
            float f[8]; uint32_t xn[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 v = bf16x2_bits_to_f32x2(xw[e]);
                if (norm) {
                    const float2 w = bf16x2_bits_to_f32x2(ww[e]);
                    // rounded to bf16 like a standalone norm kernel would store it
                    v.x = bf16_to_f32(f32_to_bf16(v.x * ir * (1.f + w.x)));
                    v.y = bf16_to_f32(f32_to_bf16(v.y * ir * (1.f + w.y)));
                } else if (gated) {
                    const float2 g = bf16x2_bits_to_f32x2(gw[e]);
                    v.x = bf16_to_f32(f32_to_bf16(v.x * sigmoid_f(g.x)));
                    v.y = bf16_to_f32(f32_to_bf16(v.y * sigmoid_f(g.y)));
                }
                xn[e] = f32x2_to_bf16x2_bits(v.x, v.y);
                f[2 * e] = v.x * s; f[2 * e + 1] = v.y * s;
            }
            if (a.xn_out != nullptr && blockIdx.x == 0 && live && idx < kvec)
                *(reinterpret_cast<uint4*>(a.xn_out + (size_t)m * a.K) + idx) = make_uint4(xn[0], xn[1], xn[2], xn[3]);
            const int k0 = idx << 3;
            if (idx < nvec) {
            if constexpr (sizeof(XS) == 4) {
                *reinterpret_cast<float4*>(xrow + xpos<WF>(k0)) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(xrow + xpos<WF>(k0 + 4)) = make_float4(f[4], f[5], f[6], f[7]);
            } else {
                uint4 h;
                __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]);
                __half2 h2 = __floats2half2_rn(f[4], f[5]), h3 = __floats2half2_rn(f[6], f[7]);
                h.x = *reinterpret_cast<uint32_t*>(&h0); h.y = *reinterpret_cast<uint32_t*>(&h1);
                h.z = *reinterpret_cast<uint32_t*>(&h2); h.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(xrow + xpos<WF>(k0)) = h;
            }
            }
        }
    }
}

// ---- packed conversions straight from 32-bit words (no per-byte shift/mask in front of the cvt)
// 8 E2M1 nibbles -> 4 half2; nibble 2j is the low half of h[j].
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(w));
}
// 4 E4M3 bytes -> 2 half2; byte 2j is the low half of h[j].
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t (&h)[2]) {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
        "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
        : "=r"(h[0]), "=r"(h[1]) : "r"(w));
}
__device__ __forceinline__ __half2 as_half2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ float half2_hsum_f32(__half2 p) { return __half2float(__hadd(__low2half(p), __high2half(p))); }

// One lane's share of one weight row inside a block: kChunk weights against one batch row's staged
// activations (`xm` = this lane's activations for that k range, as 32-bit words, shared by the rows
// of the quad; `xs` passed to load_x points at the lane's first 16-byte group of the step, see xpos).  Identical code serves the register-ring and the TMA-ring kernels.
template <int WF> struct RowDot;

template <> struct RowDot<W_BF16> {
    static constexpr int kXWords = 8;       // 8 fp32 activations
    __device__ static __forceinline__ void load_x(const float* xs, uint32_t (&xm)[kXWords]) {
        const uint4 a = *reinterpret_cast<const uint4*>(xs);
        const uint4 b = *(reinterpret_cast<const uint4*>(xs) + 32);
        xm[0] = a.x; xm[1] = a.y; xm[2] = a.z; xm[3] = a.w; xm[4] = b.x; xm[5] = b.y; xm[6] = b.z; xm[7] = b.w;
    }
    __device__ static __forceinline__ float dot(uint4 w, uint32_t /*scale_bits*/, const uint32_t (&xm)[kXWords], float acc) {
        const float2 w0 = bf16x2_bits_to_f32x2(w.x), w1 = bf16x2_bits_to_f32x2(w.y);
        const float2 w2 = bf16x2_bits_to_f32x2(w.z), w3 = bf16x2_bits_to_f32x2(w.w);
        float s = acc;
        s = fmaf(w0.x, __uint_as_float(xm[0]), s); s = fmaf(w0.y, __uint_as_float(xm[1]), s);
        s = fmaf(w1.x, __uint_as_float(xm[2]), s); s = fmaf(w1.y, __uint_as_float(xm[3]), s);
        s = fmaf(w2.x, __uint_as_float(xm[4]), s); s = fmaf(w2.y, __uint_as_float(xm[5]), s);
        s = fmaf(w3.x, __uint_as_float(xm[6]), s); s = fmaf(w3.y, __uint_as_float(xm[7]), s);
        return s;
    }
    __device__ static __forceinline__ uint32_t load_scale(const uint8_t*, int, int) { return 0u; }
};

template <> struct RowDot<W_NVFP4> {
    static constexpr int kXWords = 16;      // 32 fp16 activations
    __device__ static __forceinline__ void load_x(const __half* xs, uint32_t (&xm)[kXWords]) {
        const uint4* xp = reinterpret_cast<const uint4*>(xs);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = xp[q * 32];
            xm[q * 4] = v.x; xm[q * 4 + 1] = v.y; xm[q * 4 + 2] = v.z; xm[q * 4 + 3] = v.w;
        }
    }
    __device__ static __forceinline__ float dot(uint4 w, uint32_t scale_bits, const uint32_t (&xm)[kXWords], float acc) {
        uint32_t sh[2];
        cvt_e4m3x4(scale_bits, sh);                       // low 16 bits hold this lane's two UE4M3 scales
        const float2 sc = __half22float2(as_half2(sh[0]));
        const uint32_t wq[4] = {w.x, w.y, w.z, w.w};
        float s = acc;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            uint32_t h0[4], h1[4];
            cvt_e2m1x8(wq[2 * b], h0);
            cvt_e2m1x8(wq[2 * b + 1], h1);
            __half2 p = __hmul2(as_half2(h0[0]), as_half2(xm[b * 8 + 0]));
            p = __hfma2(as_half2(h0[1]), as_half2(xm[b * 8 + 1]), p);
            p = __hfma2(as_half2(h0[2]), as_half2(xm[b * 8 + 2]), p);
            p = __hfma2(as_half2(h0[3]), as_half2(xm[b * 8 + 3]), p);
            p = __hfma2(as_half2(h1[0]), as_half2(xm[b * 8 + 4]), p);
            p = __hfma2(as_half2(h1[1]), as_half2(xm[b * 8 + 5]), p);
            p = __hfma2(as_half2(h1[2]), as_half2(xm[b * 8 + 6]), p);
            p = __hfma2(as_half2(h1[3]), as_half2(xm[b * 8 + 7]), p);
            s = fmaf(half2_hsum_f32(p), b == 0 ? sc.x : sc.y, s);
        }
        return s;
    }
    __device__ static __forceinline__ uint32_t load_scale(const uint8_t* block, int r, int lane) {
        return *reinterpret_cast<const uint16_t*>(block + 2048 + r * 64 + lane * 2);
    }
};

template <> struct RowDot<W_MXFP8> {
    static constexpr int kXWords = 8;       // 16 fp16 activations
    __device__ static __forceinline__ void load_x(const __half* xs, uint32_t (&xm)[kXWords]) {
        const uint4* xp = reinterpret_cast<const uint4*>(xs);
        const uint4 a = xp[0], b = xp[32];
        xm[0] = a.x; xm[1] = a.y; xm[2] = a.z; xm[3] = a.w; xm[4] = b.x; xm[5] = b.y; xm[6] = b.z; xm[7] = b.w;
    }
    __device__ static __forceinline__ float dot(uint4 w, uint32_t scale_bits, const uint32_t (&xm)[kXWords], float acc) {
        const float sc = __uint_as_float(scale_bits << 23);   // UE8M0: 2^(e-127)
        const uint32_t wq[4] = {w.x, w.y, w.z, w.w};
        uint32_t h[2];
        cvt_e4m3x4(wq[0], h);
        __half2 p = __hmul2(as_half2(h[0]), as_half2(xm[0]));
        p = __hfma2(as_half2(h[1]), as_half2(xm[1]), p);
#pragma unroll
        for (int j = 1; j < 4; ++j) {
            cvt_e4m3x4(wq[j], h);
            p = __hfma2(as_half2(h[0]), as_half2(xm[2 * j]), p);
            p = __hfma2(as_half2(h[1]), as_half2(xm[2 * j + 1]), p);
        }
        return fmaf(half2_hsum_f32(p), sc, acc);
    }
    __device__ static __forceinline__ uint32_t load_scale(const uint8_t* block, int r, int lane) {
        return block[2048 + r * 16 + (lane >> 1)];
    }
};

// Apply the epilogue for one quad (4 consecutive output rows) and one batch row.
__device__ __forceinline__ void quad_epilogue(const LinearSmallArgs& a, int n0, int m, const float (&v)[kQuadRows]) {
    if (a.epilogue == EPI_SWIGLU) {
        // rows (2j, 2j+1) hold (gate_j, up_j); both rounded to bf16 as separate projections would be
#pragma unroll
        for (int h = 0; h < kQuadRows / 2; ++h) {
            if (n0 + 2 * h + 1 < a.N) {
                const float g = bf16_to_f32(f32_to_bf16(v[2 * h])), up = bf16_to_f32(f32_to_bf16(v[2 * h + 1]));
                const float y = silu_f(g) * up;
                const int j = (n0 >> 1) + h;
                if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + j] = y;
                else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + j] = f32_to_bf16(y);
            }
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < kQuadRows; ++r) {
        const int n = n0 + r;
        if (n >= a.N) continue;
        float y = v[r];
        if (a.epilogue == EPI_RESIDUAL)   // y rounded to bf16 before the add, like projection-then-add
            y = bf16_to_f32(f32_to_bf16(y)) + bf16_to_f32(a.residual[(size_t)m * a.ld_res + n]);
        if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n] = y;
        else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)m * a.ldo + n] = f32_to_bf16(y);
    }
}

// One warp's (quad, k-step) unit stream: the CTA's quads are processed in waves of at most
// `wave_max` quads; inside a wave the units are cut into `n_warps` contiguous slices.
struct QuadWalker {
    int quad_end, steps, warp, n_warps, wave_max;
    int wave_q0, wave_quads, u, u_end, q, st;     // current unit = (q, st)
    __device__ __forceinline__ void set_wave(int q0) {
        wave_q0 = q0;
        wave_quads = min(wave_max, quad_end - q0);
        if (wave_quads <= 0) { u = u_end = 0; return; }
        const int total = wave_quads * steps;
        u = (total * warp) / n_warps;
        u_end = (total * (warp + 1)) / n_warps;
        q = wave_q0 + u / steps; st = u % steps;
    }
    __device__ __forceinline__ void init(int qb, int qe, int steps_, int warp_, int n_warps_, int wave_max_) {
        quad_end = qe; steps = steps_; warp = warp_; n_warps = n_warps_; wave_max = wave_max_;
        set_wave(qb);
        while (wave_quads > 0 && u >= u_end) set_wave(wave_q0 + wave_max);
    }
    __device__ __forceinline__ bool valid() const { return wave_quads > 0; }
    __device__ __forceinline__ void next() {
        if (wave_quads <= 0) return;
        ++u;
        if (++st == steps) { st = 0; ++q; }
        while (wave_quads > 0 && u >= u_end) set_wave(wave_q0 + wave_max);
    }
};

}  // namespace ps
