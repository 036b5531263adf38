// DFlash2 block-drafter kernels: everything of a proposal that is not a projection (projections run on the
// block-scaled tensor-core kernel, gemm_bs.cu).  A proposal works on a block of T <= 16 rows
// ([anchor, MASK x K]) against a ring of up to `window` committed context rows per layer.
//
//   ps_dfl_rmsnorm        direct-weight RMSNorm, normalised value rounded to bf16 before the weight multiply
//   ps_dfl_norm_proj4     fused RMSNorm + dynamic-kernel projection + conv prepare (or + selector projection)
//   ps_dfl_conv_apply     grouped dynamic causal conv (kernel 2, block-local): prepare / finish phase (+ residual)
//   ps_dfl_headnorm_rope  per-head RMSNorm (same rounding) + full-width NeoX RoPE with bf16-rounded cos / sin
//   ps_dfl_ring_attention non-causal sliding-window GQA attention over [ring context || block rows], split over keys
//   ps_dfl_kv_ring_append per-layer k-norm + RoPE of the context keys, scatter of K / V into slot pos % window
//   ps_dfl_feature_concat the tapped target hidden states side by side: [rows, taps * H]
//   ps_dfl_noise_ids      block token ids and positions from a device control word: anchor, then K mask ids
//   ps_dfl_remap_ids      draft-vocabulary local ids -> global ids after the top-k
//   ps_dfl_select         sequential candidate selector over the top-k of every draft row
//
// Semantics follow the reference's drafter description (docs/developer/dflash2.md:221-318,363-416,496-568) and
// its kernels (src/phaseshift/models/qwen35/kernels/dflash2/{rmsnorm.hip:13-35, grouped_dynamic_conv.hip:24-65,
// rope.hip:15-39, attention.hip:283-532, kv_ring.hip:15-39, feature_concat.hip:14-53, noise_input.hip:12-24,
// candidate_selector.hip:22-91}); the kernels themselves are written for this engine's layouts.
#include "ps_common.cuh"

namespace ps {

// ---- direct-weight RMSNorm: y = bf16( bf16(x * rsqrt(mean x^2 + eps)) * w ), one CTA per row
__global__ void __launch_bounds__(256) dfl_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                          const __nv_bfloat16* __restrict__ w, float eps, int H,
                                                          __nv_bfloat16* __restrict__ out, int ldo) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const __nv_bfloat16* xr = x + (size_t)r * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x * 2; i < H; i += 512) {
        const float2 v = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + i));
        ss += v.x * v.x + v.y * v.y;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x * 2; i < H; i += 512) {
        const float2 v = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + i));
        const float2 wv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(w + i));
        const float a = bf16_to_f32(f32_to_bf16(v.x * inv)) * wv.x, b = bf16_to_f32(f32_to_bf16(v.y * inv)) * wv.y;
        *reinterpret_cast<uint32_t*>(out + (size_t)r * ldo + i) = f32x2_to_bf16x2_bits(a, b);
    }
}

// ---- grouped dynamic causal conv, one phase:
// out[t, f] = (base[phase][0][f] + dyn[t][phase][0][g]) * in[t, f] + (base[phase][1][f] + dyn[t][phase][1][g]) * in[t-1, f]
// with in[-1] = 0, g = f / group_size, dyn = kernel_projection output [T, 2 phases, 2 offsets, groups]; + residual.
__global__ void __launch_bounds__(256) dfl_conv_apply_kernel(const __nv_bfloat16* __restrict__ in, int ld_in,
                                                             const __nv_bfloat16* __restrict__ dyn, int ld_dyn,
                                                             const __nv_bfloat16* __restrict__ base, int phase, int H,
                                                             int groups, int group_size,
                                                             const __nv_bfloat16* __restrict__ residual, int ld_res,
                                                             __nv_bfloat16* __restrict__ out, int ldo) {
    const int t = blockIdx.y;
    const int f = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (f >= H) return;
    const int g = f / group_size;                      // group_size is even: both features share a group
    const __nv_bfloat16* d = dyn + (size_t)t * ld_dyn + phase * 2 * groups;
    const float d0 = bf16_to_f32(d[g]), d1 = bf16_to_f32(d[groups + g]);
    const float2 b0 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(base + ((size_t)phase * 2 + 0) * H + f));
    const float2 b1 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(base + ((size_t)phase * 2 + 1) * H + f));
    const float2 x = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(in + (size_t)t * ld_in + f));
    float2 p = make_float2(0.f, 0.f);
    if (t > 0) p = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(in + (size_t)(t - 1) * ld_in + f));
    // kernel taps and products rounded to bf16 like the tensor-op formulation they restate
    const float k0x = bf16_to_f32(f32_to_bf16(b0.x + d0)), k0y = bf16_to_f32(f32_to_bf16(b0.y + d0));
    const float k1x = bf16_to_f32(f32_to_bf16(b1.x + d1)), k1y = bf16_to_f32(f32_to_bf16(b1.y + d1));
    float ox = bf16_to_f32(f32_to_bf16(k0x * x.x)) + bf16_to_f32(f32_to_bf16(k1x * p.x));
    float oy = bf16_to_f32(f32_to_bf16(k0y * x.y)) + bf16_to_f32(f32_to_bf16(k1y * p.y));
    if (residual != nullptr) {
        const float2 r = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(residual + (size_t)t * ld_res + f));
        ox = bf16_to_f32(f32_to_bf16(ox)) + r.x; oy = bf16_to_f32(f32_to_bf16(oy)) + r.y;
    }
    *reinterpret_cast<uint32_t*>(out + (size_t)t * ldo + f) = f32x2_to_bf16x2_bits(ox, oy);
}

// ---- fused: direct RMSNorm -> tiny projection (4 C outputs per row) -> either the conv "prepare" phase or the
// normalised rows.  One launch replaces norm + projection GEMM + elementwise conv for the two places a layer needs
// them (before q/k/v and before the MLP) and norm + selector projection at the head.
// CTA c of C owns projection outputs {c, c + C, c + 2C, c + 3C} (for the dynamic conv: the four taps
// [phase][offset] of group c) and the feature slice [c H/C, (c+1) H/C) of the output rows.
//   mode 0: y[t, f] = n[t, f]                                                          (proj stored as fp32)
//   mode 1: y[t, f] = (base[0][0][f] + p[t][c]) n[t, f] + (base[0][1][f] + p[t][c + C]) n[t-1, f]   (proj stored as bf16)
// with n = bf16(bf16(x rsqrt(mean x^2 + eps)) w) and the projection accumulated in fp32 over bf16 weights.
constexpr int kDflFusedMaxRows = 16;
__device__ __forceinline__ float dfl_norm_val(float x, float inv, float w) {
    return bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(x * inv)) * w));
}
// grid (C, T): CTA (c, t) serves row t (and needs the statistics of row t - 1 for the conv's second tap)
__global__ void __launch_bounds__(256) dfl_norm_proj4_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ nw,
                                                             float eps, const __nv_bfloat16* __restrict__ wp, int C, int T, int H, int mode,
                                                             const __nv_bfloat16* __restrict__ base, void* __restrict__ proj_out, int ld_proj,
                                                             __nv_bfloat16* __restrict__ y, int ldy) {
    __shared__ float red[32 * 5];
    const int c = blockIdx.x, t = blockIdx.y;
    const bool has_prev = mode == 1 && t > 0;
    const __nv_bfloat16* xr = x + (size_t)t * ldx;
    const __nv_bfloat16* xp = x + (size_t)(has_prev ? t - 1 : t) * ldx;
    // ---- row statistics of rows t and t - 1
    float ss[2] = {0.f, 0.f};
    for (int k = threadIdx.x * 8; k < H; k += 2048) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + k);
        const uint4 v = has_prev ? *reinterpret_cast<const uint4*>(xp + k) : u;
        const uint32_t us[4] = {u.x, u.y, u.z, u.w}, vs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 a = bf16x2_bits_to_f32x2(us[e]), b = bf16x2_bits_to_f32x2(vs[e]);
            ss[0] += a.x * a.x + a.y * a.y;
            ss[1] += b.x * b.x + b.y * b.y;
        }
    }
    block_sum_n<2>(ss, red);
    const float inv = rsqrtf(ss[0] / (float)H + eps), pinv = rsqrtf(ss[1] / (float)H + eps);
    // ---- the four projection outputs of this CTA
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = threadIdx.x * 8; k < H; k += 2048) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + k);
        const uint4 wv = *reinterpret_cast<const uint4*>(nw + k);
        uint4 pv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) pv[j] = *reinterpret_cast<const uint4*>(wp + (size_t)(c + j * C) * H + k);
        const uint32_t xs[4] = {u.x, u.y, u.z, u.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
        float n[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 xv = bf16x2_bits_to_f32x2(xs[e]), w2 = bf16x2_bits_to_f32x2(ws[e]);
            n[2 * e] = dfl_norm_val(xv.x, inv, w2.x);
            n[2 * e + 1] = dfl_norm_val(xv.y, inv, w2.y);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t ps4[4] = {pv[j].x, pv[j].y, pv[j].z, pv[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 p2 = bf16x2_bits_to_f32x2(ps4[e]);
                acc[j] += n[2 * e] * p2.x + n[2 * e + 1] * p2.y;
            }
        }
    }
    block_sum_n<4>(acc, red);
    if (mode == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = bf16_to_f32(f32_to_bf16(acc[j]));       // what a bf16 projection output holds
    }
    if (threadIdx.x < 4) {
        float v = acc[0];
        if (threadIdx.x == 1) v = acc[1];
        if (threadIdx.x == 2) v = acc[2];
        if (threadIdx.x == 3) v = acc[3];
        const size_t o = (size_t)t * ld_proj + c + threadIdx.x * C;
        if (mode == 1) reinterpret_cast<__nv_bfloat16*>(proj_out)[o] = f32_to_bf16(v);
        else reinterpret_cast<float*>(proj_out)[o] = v;
    }
    // ---- output row t of this CTA's feature slice
    const int FS = H / C, f0 = c * FS;
    for (int i = threadIdx.x; i < FS / 2; i += 256) {
        const int f = f0 + i * 2;
        const float2 w2 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(nw + f));
        const float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + f));
        const float nx = dfl_norm_val(xv.x, inv, w2.x), ny = dfl_norm_val(xv.y, inv, w2.y);
        if (mode == 0) {
            *reinterpret_cast<uint32_t*>(y + (size_t)t * ldy + f) = f32x2_to_bf16x2_bits(nx, ny);
            continue;
        }
        float px = 0.f, py = 0.f;
        if (has_prev) {
            const float2 pv2 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xp + f));
            px = dfl_norm_val(pv2.x, pinv, w2.x); py = dfl_norm_val(pv2.y, pinv, w2.y);
        }
        const float2 b0 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(base + f));
        const float2 b1 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(base + H + f));
        const float k0x = bf16_to_f32(f32_to_bf16(b0.x + acc[0])), k0y = bf16_to_f32(f32_to_bf16(b0.y + acc[0]));
        const float k1x = bf16_to_f32(f32_to_bf16(b1.x + acc[1])), k1y = bf16_to_f32(f32_to_bf16(b1.y + acc[1]));
        const float ox = bf16_to_f32(f32_to_bf16(k0x * nx)) + bf16_to_f32(f32_to_bf16(k1x * px));
        const float oy = bf16_to_f32(f32_to_bf16(k0y * ny)) + bf16_to_f32(f32_to_bf16(k1y * py));
        *reinterpret_cast<uint32_t*>(y + (size_t)t * ldy + f) = f32x2_to_bf16x2_bits(ox, oy);
    }
}

// ---- per-head RMSNorm (direct weight) + NeoX RoPE over the whole head; one warp per (row, head), D <= 256
__device__ __forceinline__ void headnorm_rope_row(const __nv_bfloat16* src, const __nv_bfloat16* w, float eps, int D,
                                                  float pos, float theta, bool do_norm, __nv_bfloat16* dst, int lane) {
    const int half = D >> 1;
    float lo[4], hi[4];                                 // element (lane + 32 j) of each half
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        lo[j] = i < half ? bf16_to_f32(src[i]) : 0.f;
        hi[j] = i < half ? bf16_to_f32(src[half + i]) : 0.f;
        ss += lo[j] * lo[j] + hi[j] * hi[j];
    }
    ss = warp_sum(ss);
    const float inv = do_norm ? rsqrtf(ss / (float)D + eps) : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        if (i >= half) continue;
        float a = lo[j], b = hi[j];
        if (do_norm) {
            a = bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(a * inv)) * bf16_to_f32(w[i])));
            b = bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(b * inv)) * bf16_to_f32(w[half + i])));
        }
        const float inv_freq = powf(theta, -(float)(2 * i) / (float)D);
        const float ang = pos * inv_freq;
        const float c = bf16_to_f32(f32_to_bf16(cosf(ang))), s = bf16_to_f32(f32_to_bf16(sinf(ang)));
        // products and sums rounded like bf16 tensor arithmetic
        dst[i] = f32_to_bf16(bf16_to_f32(f32_to_bf16(a * c)) - bf16_to_f32(f32_to_bf16(b * s)));
        dst[half + i] = f32_to_bf16(bf16_to_f32(f32_to_bf16(b * c)) + bf16_to_f32(f32_to_bf16(a * s)));
    }
}

__global__ void __launch_bounds__(128) dfl_headnorm_rope_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int heads, int D,
                                                                const __nv_bfloat16* __restrict__ w, int heads_w,
                                                                const __nv_bfloat16* __restrict__ w2, float eps,
                                                                const int* __restrict__ pos, float theta, int rows,
                                                                __nv_bfloat16* __restrict__ out, int ldo) {
    const int wid = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wid >= rows * heads) return;
    const int t = wid / heads, h = wid - t * heads;
    // heads [0, heads_w) take weight w (queries), the rest w2 (keys of a fused q|k projection)
    headnorm_rope_row(x + (size_t)t * ldx + h * D, h < heads_w ? w : w2, eps, D, (float)pos[t], theta, true,
                      out + (size_t)t * ldo + h * D, lane);
}

// ---- context append: kv [n, layers * 2 * kvf] (per layer [k | v]) -> rings [layers, window, kvf]
__global__ void __launch_bounds__(128) dfl_kv_ring_append_kernel(const __nv_bfloat16* __restrict__ kv, int ld, int layers,
                                                                 int kv_heads, int D, const __nv_bfloat16* __restrict__ k_norm_w,
                                                                 float eps, int pos_start, int window, float theta, int n,
                                                                 __nv_bfloat16* __restrict__ k_ring, __nv_bfloat16* __restrict__ v_ring,
                                                                 int* __restrict__ ring_pos, const int* __restrict__ ctl) {
    const int wid = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int kvf = kv_heads * D;
    if (ctl != nullptr) { n = min(n, ctl[1]); pos_start = ctl[3]; }      // {-, rows to keep, -, first position} on the device
    if (wid >= n * layers * kv_heads) return;
    const int h = wid % kv_heads, l = (wid / kv_heads) % layers, r = wid / (kv_heads * layers);
    const int pos = pos_start + r, slot = pos % window;
    const __nv_bfloat16* src = kv + (size_t)r * ld + (size_t)l * 2 * kvf;
    __nv_bfloat16* kd = k_ring + ((size_t)l * window + slot) * kvf + h * D;
    __nv_bfloat16* vd = v_ring + ((size_t)l * window + slot) * kvf + h * D;
    headnorm_rope_row(src + h * D, k_norm_w + (size_t)l * D, eps, D, (float)pos, theta, true, kd, lane);
    for (int i = lane; i < D; i += 32) vd[i] = src[kvf + h * D + i];
    if (l == 0 && h == 0 && lane == 0) ring_pos[slot] = pos;
}

// ---- ring GQA attention, split over the keys.
// Keys = the `window` ring slots followed by the block's own T rows; mask: slot filled and |pos_q - pos_k| < window;
// non-causal.  Launch 1: one CTA per (64-key tile, kv head) scores ALL query rows of that kv head (T rows x G heads
// <= 64) against its tile -- every K / V byte is read once -- and writes an unnormalised partial (o, max, sum) per
// row.  Launch 2 merges the partials of a (row, head).  Register-blocked fp32 FMA: the whole op is ~0.3 GFLOP.
constexpr int kDflKT = 64;            // keys per CTA
constexpr int kDflQMax = 64;          // query rows (T * G) per kv head
constexpr int kDflKPitch = 132;       // bf16 per Q / K row in shared memory: 8-byte aligned, conflict-free 8-byte column reads
constexpr int kDflVPitch = 136;       // bf16 per V row: 16-byte aligned
constexpr int kDflPPitch = 65;        // fp32 per probability row
constexpr int kDflPartLd = 132;       // fp32 per partial row: 128 outputs, running max, running sum, 2 pad
constexpr int kDflAttnSmem = (2 * kDflKT * kDflKPitch + kDflKT * kDflVPitch) * 2 + kDflQMax * kDflPPitch * 4 + 2 * 64 * 4;

__device__ __forceinline__ void unpack4(const uint2 u, float (&f)[4]) {
    const float2 a = bf16x2_bits_to_f32x2(u.x), b = bf16x2_bits_to_f32x2(u.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

template <int QR>      // query rows per thread: 2 serves up to 32 rows, 4 up to 64
__global__ void __launch_bounds__(256) dfl_ring_attention_split_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                                                                       const __nv_bfloat16* __restrict__ kb, const __nv_bfloat16* __restrict__ vb, int ldkv,
                                                                       const __nv_bfloat16* __restrict__ k_ring, const __nv_bfloat16* __restrict__ v_ring,
                                                                       const int* __restrict__ ring_pos, const int* __restrict__ pos,
                                                                       int T, int window, int G, int kv_heads, float scale,
                                                                       float* __restrict__ part) {
    constexpr int D = 128;
    extern __shared__ __align__(16) unsigned char dfl_smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dfl_smem);
    __nv_bfloat16* sK = sQ + kDflQMax * kDflKPitch;
    __nv_bfloat16* sV = sK + kDflKT * kDflKPitch;
    float* sP = reinterpret_cast<float*>(sV + kDflKT * kDflVPitch);
    int* sPos = reinterpret_cast<int*>(sP + kDflQMax * kDflPPitch);
    int* sQpos = sPos + 64;
    const int split = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x;
    const int kvf = kv_heads * D, Q = T * G, total = window + T, k0 = split * kDflKT;
    // ---- stage Q (all rows of this kv head), the K / V tile and the positions
    for (int i = tid; i < 16 * QR * (D / 4); i += 256) {
        const int r = i / (D / 4), c = i - r * (D / 4);
        uint2 v = make_uint2(0u, 0u);
        if (r < Q) { const int t = r / G, g = r - t * G; v = *reinterpret_cast<const uint2*>(q + (size_t)t * ldq + (kvh * G + g) * D + c * 4); }
        *reinterpret_cast<uint2*>(sQ + r * kDflKPitch + c * 4) = v;
    }
    for (int i = tid; i < kDflKT * (D / 4); i += 256) {
        const int r = i / (D / 4), c = i - r * (D / 4), key = k0 + r;
        uint2 v = make_uint2(0u, 0u);
        if (key < window) v = *reinterpret_cast<const uint2*>(k_ring + (size_t)key * kvf + kvh * D + c * 4);
        else if (key < total) v = *reinterpret_cast<const uint2*>(kb + (size_t)(key - window) * ldkv + kvh * D + c * 4);
        *reinterpret_cast<uint2*>(sK + r * kDflKPitch + c * 4) = v;
    }
    for (int i = tid; i < kDflKT * (D / 8); i += 256) {
        const int r = i / (D / 8), c = i - r * (D / 8), key = k0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (key < window) v = *reinterpret_cast<const uint4*>(v_ring + (size_t)key * kvf + kvh * D + c * 8);
        else if (key < total) v = *reinterpret_cast<const uint4*>(vb + (size_t)(key - window) * ldkv + kvh * D + c * 8);
        *reinterpret_cast<uint4*>(sV + r * kDflVPitch + c * 8) = v;
    }
    if (tid < kDflKT) {
        const int key = k0 + tid;
        sPos[tid] = key < window ? ring_pos[key] : (key < total ? pos[key - window] : -1);
        sQpos[tid] = tid < Q ? pos[tid / G] : 0;
    }
    __syncthreads();
    // ---- scores: thread (tq, tk) owns rows tq * QR + i and keys tk + 16 j
    const int tq = tid >> 4, tk = tid & 15;
    float acc[QR][4];
#pragma unroll
    for (int i = 0; i < QR; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int c = 0; c < D / 4; ++c) {
        float qf[QR][4], kf[4][4];
#pragma unroll
        for (int i = 0; i < QR; ++i) unpack4(*reinterpret_cast<const uint2*>(sQ + (tq * QR + i) * kDflKPitch + c * 4), qf[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack4(*reinterpret_cast<const uint2*>(sK + (tk + 16 * j) * kDflKPitch + c * 4), kf[j]);
#pragma unroll
        for (int i = 0; i < QR; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                acc[i][j] += qf[i][0] * kf[j][0] + qf[i][1] * kf[j][1] + qf[i][2] * kf[j][2] + qf[i][3] * kf[j][3];
    }
    float* prt = part + ((size_t)split * kv_heads + kvh) * kDflQMax * kDflPartLd;
#pragma unroll
    for (int i = 0; i < QR; ++i) {
        const int row = tq * QR + i, pq = sQpos[row];
        float sc[4], mx = -3.0e38f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kp = sPos[tk + 16 * j];
            const bool ok = kp >= 0 && abs(pq - kp) < window;
            sc[j] = ok ? acc[i][j] * scale : -3.0e38f;
            mx = fmaxf(mx, sc[j]);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));     // the 16 lanes of one tq
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float p = sc[j] > -3.0e38f ? __expf(sc[j] - mx) : 0.f;
            sP[row * kDflPPitch + tk + 16 * j] = p;
            sum += p;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (tk == 0 && row < Q) { prt[(size_t)row * kDflPartLd + D] = mx; prt[(size_t)row * kDflPartLd + D + 1] = sum; }
    }
    __syncthreads();
    // ---- partial outputs: thread (tq, tk) owns rows tq * QR + i and dims 8 tk .. 8 tk + 7
    float o[QR][8];
#pragma unroll
    for (int i = 0; i < QR; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) o[i][e] = 0.f;
#pragma unroll 4
    for (int key = 0; key < kDflKT; ++key) {
        const uint4 vv = *reinterpret_cast<const uint4*>(sV + key * kDflVPitch + tk * 8);
        float vf[8];
        { const float2 a = bf16x2_bits_to_f32x2(vv.x), b = bf16x2_bits_to_f32x2(vv.y), c2 = bf16x2_bits_to_f32x2(vv.z), d2 = bf16x2_bits_to_f32x2(vv.w);
          vf[0] = a.x; vf[1] = a.y; vf[2] = b.x; vf[3] = b.y; vf[4] = c2.x; vf[5] = c2.y; vf[6] = d2.x; vf[7] = d2.y; }
#pragma unroll
        for (int i = 0; i < QR; ++i) {
            const float p = sP[(tq * QR + i) * kDflPPitch + key];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[i][e] += p * vf[e];
        }
    }
#pragma unroll
    for (int i = 0; i < QR; ++i) {
        const int row = tq * QR + i;
        if (row >= Q) continue;
        float4* dst = reinterpret_cast<float4*>(prt + (size_t)row * kDflPartLd + tk * 8);
        dst[0] = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
        dst[1] = make_float4(o[i][4], o[i][5], o[i][6], o[i][7]);
    }
}

// merge the per-tile partials of one (block row, query head): grid T * q_heads, 128 threads (one per dim)
__global__ void __launch_bounds__(128) dfl_ring_attention_merge_kernel(const float* __restrict__ part, int splits, int G, int kv_heads,
                                                                       int q_heads, __nv_bfloat16* __restrict__ out, int ldo) {
    constexpr int D = 128;
    const int t = blockIdx.x / q_heads, h = blockIdx.x - t * q_heads;
    const int kvh = h / G, row = t * G + (h - kvh * G), d = threadIdx.x;
    const size_t stride = (size_t)kv_heads * kDflQMax * kDflPartLd;
    const float* p0 = part + ((size_t)kvh * kDflQMax + row) * kDflPartLd;
    float M = -3.0e38f;
    for (int s2 = 0; s2 < splits; ++s2) M = fmaxf(M, p0[s2 * stride + D]);
    float L = 0.f, acc = 0.f;
    for (int s2 = 0; s2 < splits; ++s2) {
        const float ms = p0[s2 * stride + D];
        if (ms <= -3.0e38f) continue;
        const float w = __expf(ms - M);
        L += w * p0[s2 * stride + D + 1];
        acc += w * p0[s2 * stride + d];
    }
    out[(size_t)t * ldo + h * D + d] = f32_to_bf16(L > 0.f ? acc / L : 0.f);
}

struct DflConcatArgs { const __nv_bfloat16* src[8]; int ld[8]; int n; };
__global__ void __launch_bounds__(256) dfl_feature_concat_kernel(const DflConcatArgs a, int rows, int H, __nv_bfloat16* __restrict__ out) {
    const int r = blockIdx.y, tp = blockIdx.z;
    const uint4* s = reinterpret_cast<const uint4*>(a.src[tp] + (size_t)r * a.ld[tp]);
    uint4* d = reinterpret_cast<uint4*>(out + ((size_t)r * a.n + tp) * H);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H / 8; i += gridDim.x * blockDim.x) d[i] = s[i];
}

// ctl = {anchor token, first position} on the device: a captured graph replays with new values
__global__ void dfl_noise_ids_kernel(const int* __restrict__ ctl, int mask_id, int k, int* __restrict__ ids, int* __restrict__ pos) {
    const int i = threadIdx.x;
    if (i > k) return;
    ids[i] = i == 0 ? ctl[0] : mask_id;
    pos[i] = ctl[1] + i;
}

// local -> global token ids after a top-k over a draft-vocabulary subset (-1 stays -1)
__global__ void dfl_remap_ids_kernel(int* __restrict__ ids, int n, const int* __restrict__ idmap, int n_map) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int v = ids[i];
    ids[i] = (v >= 0 && v < n_map) ? idmap[v] : -1;
}

// ---- sequential candidate selector: one CTA walks the draft rows; for row r every candidate j of its top-kk list gets
// score_j = logit_j + sum_i pred_cb[prev][i] * hproj[r][i] * succ_cb[cand_j][i]; the best-ranked maximal candidate wins and
// becomes `prev` of the next row.  The candidates of ALL rows are known up front, so their codebook rows are staged in
// shared memory first; only pred_cb[prev] is a dependent load per row.
__global__ void __launch_bounds__(256) dfl_select_kernel(const int* __restrict__ top_ids, const float* __restrict__ top_logits, int kk,
                                                         const float* __restrict__ hproj, int rank,
                                                         const __nv_bfloat16* __restrict__ pred_cb, const __nv_bfloat16* __restrict__ succ_cb,
                                                         const int* __restrict__ anchor, int anchor_value, int K, int vocab,
                                                         int* __restrict__ out_tokens, int staged) {
    extern __shared__ __align__(16) unsigned char sel_smem[];
    __nv_bfloat16* s_succ = reinterpret_cast<__nv_bfloat16*>(sel_smem);            // [K * kk][rank] when staged
    __shared__ float s_u[256];          // pred_cb[prev] * hproj[r]
    __shared__ float s_score[128];
    __shared__ int s_prev;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) s_prev = anchor != nullptr ? anchor[0] : anchor_value;
    if (staged) {
        for (int i = threadIdx.x; i < K * kk * rank; i += 256) {
            const int cj = i / rank, cand = top_ids[cj];
            s_succ[i] = (cand >= 0 && cand < vocab) ? succ_cb[(size_t)cand * rank + (i - cj * rank)] : f32_to_bf16(0.f);
        }
    }
    __syncthreads();
    for (int r = 0; r < K; ++r) {
        const int prev = min(max(s_prev, 0), vocab - 1);
        for (int i = threadIdx.x; i < rank; i += 256) s_u[i] = bf16_to_f32(pred_cb[(size_t)prev * rank + i]) * hproj[(size_t)r * rank + i];
        __syncthreads();
        for (int j = warp; j < kk; j += 8) {
            const int cand = top_ids[r * kk + j];
            float acc = 0.f;
            if (cand >= 0 && cand < vocab) {
                const __nv_bfloat16* sr = staged ? s_succ + (size_t)(r * kk + j) * rank : succ_cb + (size_t)cand * rank;
                for (int i = lane; i < rank; i += 32) acc += s_u[i] * bf16_to_f32(sr[i]);
            }
            acc = warp_sum(acc);
            if (lane == 0) s_score[j] = cand >= 0 ? top_logits[r * kk + j] + acc : -3.0e38f;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int best = 0;
            for (int j = 1; j < kk; ++j) if (s_score[j] > s_score[best]) best = j;      // first maximum = best-ranked on ties
            s_prev = top_ids[r * kk + best];
            out_tokens[r] = s_prev;
        }
        __syncthreads();
    }
}

}  // namespace ps

PS_API int ps_dfl_rmsnorm(const void* x, int ldx, const void* w, float eps, int rows, int H, void* out, int ldo, cudaStream_t stream) {
    if (rows <= 0 || (H & 1)) return (int)cudaErrorInvalidValue;
    ps::dfl_rmsnorm_kernel<<<rows, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, eps, H, (__nv_bfloat16*)out, ldo);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_conv_apply(const void* in, int ld_in, const void* dyn, int ld_dyn, const void* base, int phase, int rows, int H,
                             int groups, const void* residual, int ld_res, void* out, int ldo, cudaStream_t stream) {
    if (rows <= 0 || H % groups || ((H / groups) & 1) || phase < 0 || phase > 1) return (int)cudaErrorInvalidValue;
    dim3 grid((H / 2 + 255) / 256, rows);
    ps::dfl_conv_apply_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)in, ld_in, (const __nv_bfloat16*)dyn, ld_dyn,
                                                        (const __nv_bfloat16*)base, phase, H, groups, H / groups,
                                                        (const __nv_bfloat16*)residual, ld_res, (__nv_bfloat16*)out, ldo);
    return PS_LAUNCH_CHECK();
}

// x [T, H] -> y [T, H] and proj [T, 4 C]; see dfl_norm_proj4_kernel.  wp: bf16 [4 C, H] row-major.
// mode 1 (conv prepare): C = conv groups, base = base_kernel [2 phases][2 offsets][H], proj_out bf16.
// mode 0 (norm + projection): proj_out fp32.
PS_API int ps_dfl_norm_proj4(const void* x, int ldx, const void* norm_w, float eps, const void* wp, int C, int T, int H, int mode,
                             const void* base, void* proj_out, int ld_proj, void* y, int ldy, cudaStream_t stream) {
    if (T < 1 || T > ps::kDflFusedMaxRows || C < 1 || H % C || ((H / C) & 1) || (H % 8) || (ldx % 8) || ((uintptr_t)x % 16) ||
        ((uintptr_t)wp % 16) || ((uintptr_t)norm_w % 16) || (mode == 1 && base == nullptr) || mode < 0 || mode > 1)
        return (int)cudaErrorInvalidValue;
    ps::dfl_norm_proj4_kernel<<<dim3(C, T), 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)norm_w, eps, (const __nv_bfloat16*)wp, C,
                                                     T, H, mode, (const __nv_bfloat16*)base, proj_out, ld_proj, (__nv_bfloat16*)y, ldy);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_headnorm_rope(const void* x, int ldx, int heads, int D, const void* w, int heads_w, const void* w2, float eps,
                                const void* pos, float theta, int rows, void* out, int ldo, cudaStream_t stream) {
    if (rows <= 0 || D > 256 || (D & 1) || (heads_w < heads && w2 == nullptr)) return (int)cudaErrorInvalidValue;
    const int warps = rows * heads;
    ps::dfl_headnorm_rope_kernel<<<(warps + 3) / 4, 128, 0, stream>>>((const __nv_bfloat16*)x, ldx, heads, D, (const __nv_bfloat16*)w, heads_w,
                                                                       (const __nv_bfloat16*)w2, eps, (const int*)pos, theta, rows, (__nv_bfloat16*)out, ldo);
    return PS_LAUNCH_CHECK();
}

// ctl (optional, int32[4] on the device): rows beyond ctl[1] are skipped and ctl[3] replaces pos_start, so that a captured
// graph can commit a number of rows that is only known on the device side of the launch.
PS_API int ps_dfl_kv_ring_append(const void* kv, int ld, int layers, int kv_heads, int D, const void* k_norm_w, float eps, int pos_start,
                                 int window, float theta, int n, void* k_ring, void* v_ring, void* ring_pos, const void* ctl,
                                 cudaStream_t stream) {
    if (n <= 0 || D > 256 || (D & 1)) return (int)cudaErrorInvalidValue;
    const int warps = n * layers * kv_heads;
    ps::dfl_kv_ring_append_kernel<<<(warps + 3) / 4, 128, 0, stream>>>((const __nv_bfloat16*)kv, ld, layers, kv_heads, D,
                                                                        (const __nv_bfloat16*)k_norm_w, eps, pos_start, window, theta, n,
                                                                        (__nv_bfloat16*)k_ring, (__nv_bfloat16*)v_ring, (int*)ring_pos,
                                                                        (const int*)ctl);
    return PS_LAUNCH_CHECK();
}

// Rows of fp32 workspace (kDflPartLd = 132 floats each) the attention needs for T block rows over `window` slots.
PS_API long long ps_dfl_ring_attention_workspace_floats(int T, int window, int kv_heads) {
    const long long splits = (window + T + ps::kDflKT - 1) / ps::kDflKT;
    return splits * kv_heads * ps::kDflQMax * ps::kDflPartLd;
}

PS_API int ps_dfl_ring_attention(const void* q, int ldq, const void* kb, const void* vb, int ldkv, const void* k_ring, const void* v_ring,
                                 const void* ring_pos, const void* pos, int T, int window, int q_heads, int kv_heads, int D, float scale,
                                 void* out, int ldo, void* workspace, cudaStream_t stream) {
    using namespace ps;
    if (T <= 0 || D != 128 || q_heads % kv_heads || (ldkv % 8) || (ldq % 4) || workspace == nullptr) return (int)cudaErrorInvalidValue;
    const int G = q_heads / kv_heads;
    if (T * G > kDflQMax) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(dfl_ring_attention_split_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDflAttnSmem);
        cudaFuncSetAttribute(dfl_ring_attention_split_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDflAttnSmem);
        attr_set = true;
    }
    const int splits = (window + T + kDflKT - 1) / kDflKT;
    dim3 grid(splits, kv_heads);
    if (T * G <= 32)
        dfl_ring_attention_split_kernel<2><<<grid, 256, kDflAttnSmem, stream>>>((const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kb, (const __nv_bfloat16*)vb, ldkv,
            (const __nv_bfloat16*)k_ring, (const __nv_bfloat16*)v_ring, (const int*)ring_pos, (const int*)pos, T, window, G, kv_heads, scale, (float*)workspace);
    else
        dfl_ring_attention_split_kernel<4><<<grid, 256, kDflAttnSmem, stream>>>((const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kb, (const __nv_bfloat16*)vb, ldkv,
            (const __nv_bfloat16*)k_ring, (const __nv_bfloat16*)v_ring, (const int*)ring_pos, (const int*)pos, T, window, G, kv_heads, scale, (float*)workspace);
    dfl_ring_attention_merge_kernel<<<T * q_heads, 128, 0, stream>>>((const float*)workspace, splits, G, kv_heads, q_heads, (__nv_bfloat16*)out, ldo);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_feature_concat(const void* const* srcs, const int* lds, int n_taps, int rows, int H, void* out, cudaStream_t stream) {
    if (rows <= 0 || n_taps < 1 || n_taps > 8 || (H % 8)) return (int)cudaErrorInvalidValue;
    ps::DflConcatArgs a;
    a.n = n_taps;
    for (int i = 0; i < 8; ++i) { a.src[i] = i < n_taps ? (const __nv_bfloat16*)srcs[i] : nullptr; a.ld[i] = i < n_taps ? lds[i] : 0; }
    dim3 grid((H / 8 + 255) / 256, rows, n_taps);
    ps::dfl_feature_concat_kernel<<<grid, 256, 0, stream>>>(a, rows, H, (__nv_bfloat16*)out);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_noise_ids(const void* ctl, int mask_id, int k, void* ids, void* pos, cudaStream_t stream) {
    if (k < 0 || k > 31 || ctl == nullptr) return (int)cudaErrorInvalidValue;
    ps::dfl_noise_ids_kernel<<<1, 32, 0, stream>>>((const int*)ctl, mask_id, k, (int*)ids, (int*)pos);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_select(const void* top_ids, const void* top_logits, int kk, const void* hproj, int rank, const void* pred_cb,
                         const void* succ_cb, const void* anchor_dev, int anchor_value, int K, int vocab, void* out_tokens,
                         cudaStream_t stream) {
    if (K <= 0 || kk < 1 || kk > 128 || rank < 1 || rank > 256) return (int)cudaErrorInvalidValue;
    const size_t stage_bytes = (size_t)K * kk * rank * 2;
    const int staged = stage_bytes <= 96 * 1024 ? 1 : 0;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(ps::dfl_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        attr_set = true;
    }
    ps::dfl_select_kernel<<<1, 256, staged ? stage_bytes : 0, stream>>>((const int*)top_ids, (const float*)top_logits, kk, (const float*)hproj, rank,
                                                                       (const __nv_bfloat16*)pred_cb, (const __nv_bfloat16*)succ_cb, (const int*)anchor_dev,
                                                                       anchor_value, K, vocab, (int*)out_tokens, staged);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_remap_ids(void* ids, int n, const void* idmap, int n_map, cudaStream_t stream) {
    if (n <= 0 || idmap == nullptr) return (int)cudaErrorInvalidValue;
    ps::dfl_remap_ids_kernel<<<(n + 255) / 256, 256, 0, stream>>>((int*)ids, n, (const int*)idmap, n_map);
    return PS_LAUNCH_CHECK();
}
