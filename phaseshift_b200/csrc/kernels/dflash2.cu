// DFlash2 block-drafter kernels: everything of a proposal that is not a projection (projections run on the
// block-scaled tensor-core kernel, gemm_bs.cu).  A proposal works on a block of T <= 16 rows
// ([anchor, MASK x K]) against a ring of up to `window` committed context rows per layer.
//
//   ps_dfl_rmsnorm        direct-weight RMSNorm, normalised value rounded to bf16 before the weight multiply
//   ps_dfl_conv_apply     grouped dynamic causal conv (kernel 2, block-local): prepare / finish phase (+ residual)
//   ps_dfl_headnorm_rope  per-head RMSNorm (same rounding) + full-width NeoX RoPE with bf16-rounded cos / sin
//   ps_dfl_ring_attention non-causal sliding-window GQA attention over [ring context || block rows]
//   ps_dfl_kv_ring_append per-layer k-norm + RoPE of the context keys, scatter of K / V into slot pos % window
//   ps_dfl_feature_concat the tapped target hidden states side by side: [rows, taps * H]
//   ps_dfl_noise_ids      block token ids and positions from a device control word: anchor, then K mask ids
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
                                                                 int* __restrict__ ring_pos) {
    const int wid = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int kvf = kv_heads * D;
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

// ---- ring GQA attention: one CTA per (block row t, kv head); warp w serves query head kvh * G + w (G <= 4).
// Keys: ring slots with ring_pos >= 0, then the block's own rows; mask |pos_q - pos_k| < window; non-causal.
constexpr int kDflKeys = 64, kDflPitch = 136;      // 64-key tiles, row pitch in bf16 (272 B: conflict-free column reads)
__global__ void __launch_bounds__(128) dfl_ring_attention_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                                                                 const __nv_bfloat16* __restrict__ kb, const __nv_bfloat16* __restrict__ vb, int ldkv,
                                                                 const __nv_bfloat16* __restrict__ k_ring, const __nv_bfloat16* __restrict__ v_ring,
                                                                 const int* __restrict__ ring_pos, const int* __restrict__ pos,
                                                                 int T, int window, int q_heads, int kv_heads, float scale,
                                                                 __nv_bfloat16* __restrict__ out, int ldo) {
    constexpr int D = 128;
    __shared__ __align__(16) __nv_bfloat16 sK[kDflKeys * kDflPitch], sV[kDflKeys * kDflPitch];
    __shared__ float sQ[4][D];
    __shared__ int sPos[kDflKeys];
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int G = q_heads / kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvf = kv_heads * D;
    const int pq = pos[t];
    if (warp < G)
        for (int i = lane; i < D; i += 32) sQ[warp][i] = bf16_to_f32(q[(size_t)t * ldq + (kvh * G + warp) * D + i]) * scale;
    float m_run = -3.0e38f, l_run = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};      // lane owns dims 4 lane .. 4 lane + 3
    const int total = window + T;
    for (int k0 = 0; k0 < total; k0 += kDflKeys) {
        __syncthreads();
        // stage a tile of keys / values (16 bytes per thread and row piece) and their positions
        for (int i = threadIdx.x; i < kDflKeys * (D / 8); i += 128) {
            const int r = i / (D / 8), c = i - r * (D / 8);
            const int key = k0 + r;
            uint4 kvv = make_uint4(0, 0, 0, 0), vvv = kvv;
            if (key < window) {
                kvv = *reinterpret_cast<const uint4*>(k_ring + (size_t)key * kvf + kvh * D + c * 8);
                vvv = *reinterpret_cast<const uint4*>(v_ring + (size_t)key * kvf + kvh * D + c * 8);
            } else if (key < total) {
                kvv = *reinterpret_cast<const uint4*>(kb + (size_t)(key - window) * ldkv + kvh * D + c * 8);
                vvv = *reinterpret_cast<const uint4*>(vb + (size_t)(key - window) * ldkv + kvh * D + c * 8);
            }
            *reinterpret_cast<uint4*>(sK + r * kDflPitch + c * 8) = kvv;
            *reinterpret_cast<uint4*>(sV + r * kDflPitch + c * 8) = vvv;
        }
        if (threadIdx.x < kDflKeys) {
            const int key = k0 + threadIdx.x;
            sPos[threadIdx.x] = key < window ? ring_pos[key] : (key < total ? pos[key - window] : -1);
        }
        __syncthreads();
        if (warp >= G) continue;
        // scores of this warp's query head: lane handles keys lane and lane + 32 of the tile
        float sc[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int r = lane + 32 * u, kp = sPos[r];
            const bool ok = kp >= 0 && abs(pq - kp) < window;
            float acc = 0.f;
            const __nv_bfloat16* kr = sK + r * kDflPitch;
#pragma unroll 8
            for (int d = 0; d < D; d += 2) {
                const float2 kv2 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(kr + d));
                acc += sQ[warp][d] * kv2.x + sQ[warp][d + 1] * kv2.y;
            }
            sc[u] = ok ? acc : -3.0e38f;
        }
        const float tmax = warp_max(fmaxf(sc[0], sc[1]));
        if (tmax <= -3.0e38f) continue;                     // the whole tile is masked
        const float m_new = fmaxf(m_run, tmax), corr = __expf(m_run - m_new);
        float p[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) p[u] = sc[u] > -3.0e38f ? __expf(sc[u] - m_new) : 0.f;
        l_run = l_run * corr + warp_sum(p[0] + p[1]);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] *= corr;
        m_run = m_new;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            for (int src = 0; src < 32; ++src) {
                const float pk = __shfl_sync(0xffffffffu, p[u], src);
                if (pk == 0.f) continue;
                const __nv_bfloat16* vr = sV + (src + 32 * u) * kDflPitch + lane * 4;
                const float2 v01 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(vr));
                const float2 v23 = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(vr + 2));
                o[0] += pk * v01.x; o[1] += pk * v01.y; o[2] += pk * v23.x; o[3] += pk * v23.y;
            }
        }
    }
    if (warp < G) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* od = out + (size_t)t * ldo + (kvh * G + warp) * D + lane * 4;
        *reinterpret_cast<uint32_t*>(od) = f32x2_to_bf16x2_bits(o[0] * inv, o[1] * inv);
        *reinterpret_cast<uint32_t*>(od + 2) = f32x2_to_bf16x2_bits(o[2] * inv, o[3] * inv);
    }
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

// ---- sequential candidate selector: one CTA walks the draft rows; for row r every candidate j of its top-kk list gets
// score_j = logit_j + sum_i pred_cb[prev][i] * hproj[r][i] * succ_cb[cand_j][i]; the best-ranked maximal candidate wins and
// becomes `prev` of the next row.
__global__ void __launch_bounds__(128) dfl_select_kernel(const int* __restrict__ top_ids, const float* __restrict__ top_logits, int kk,
                                                         const float* __restrict__ hproj, int rank,
                                                         const __nv_bfloat16* __restrict__ pred_cb, const __nv_bfloat16* __restrict__ succ_cb,
                                                         const int* __restrict__ anchor, int anchor_value, int K, int vocab,
                                                         int* __restrict__ out_tokens) {
    __shared__ float s_u[256];          // pred_cb[prev] * hproj[r]
    __shared__ float s_score[128];
    __shared__ int s_prev;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) s_prev = anchor != nullptr ? anchor[0] : anchor_value;
    __syncthreads();
    for (int r = 0; r < K; ++r) {
        const int prev = min(max(s_prev, 0), vocab - 1);
        for (int i = threadIdx.x; i < rank; i += 128) s_u[i] = bf16_to_f32(pred_cb[(size_t)prev * rank + i]) * hproj[(size_t)r * rank + i];
        __syncthreads();
        for (int j = warp; j < kk; j += 4) {
            const int cand = top_ids[r * kk + j];
            float acc = 0.f;
            if (cand >= 0 && cand < vocab)
                for (int i = lane; i < rank; i += 32) acc += s_u[i] * bf16_to_f32(succ_cb[(size_t)cand * rank + i]);
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

PS_API int ps_dfl_headnorm_rope(const void* x, int ldx, int heads, int D, const void* w, int heads_w, const void* w2, float eps,
                                const void* pos, float theta, int rows, void* out, int ldo, cudaStream_t stream) {
    if (rows <= 0 || D > 256 || (D & 1) || (heads_w < heads && w2 == nullptr)) return (int)cudaErrorInvalidValue;
    const int warps = rows * heads;
    ps::dfl_headnorm_rope_kernel<<<(warps + 3) / 4, 128, 0, stream>>>((const __nv_bfloat16*)x, ldx, heads, D, (const __nv_bfloat16*)w, heads_w,
                                                                       (const __nv_bfloat16*)w2, eps, (const int*)pos, theta, rows, (__nv_bfloat16*)out, ldo);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_kv_ring_append(const void* kv, int ld, int layers, int kv_heads, int D, const void* k_norm_w, float eps, int pos_start,
                                 int window, float theta, int n, void* k_ring, void* v_ring, void* ring_pos, cudaStream_t stream) {
    if (n <= 0 || D > 256 || (D & 1)) return (int)cudaErrorInvalidValue;
    const int warps = n * layers * kv_heads;
    ps::dfl_kv_ring_append_kernel<<<(warps + 3) / 4, 128, 0, stream>>>((const __nv_bfloat16*)kv, ld, layers, kv_heads, D,
                                                                        (const __nv_bfloat16*)k_norm_w, eps, pos_start, window, theta, n,
                                                                        (__nv_bfloat16*)k_ring, (__nv_bfloat16*)v_ring, (int*)ring_pos);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_dfl_ring_attention(const void* q, int ldq, const void* kb, const void* vb, int ldkv, const void* k_ring, const void* v_ring,
                                 const void* ring_pos, const void* pos, int T, int window, int q_heads, int kv_heads, int D, float scale,
                                 void* out, int ldo, cudaStream_t stream) {
    if (T <= 0 || D != 128 || q_heads % kv_heads || q_heads / kv_heads > 4 || (ldkv % 8) || (ldq % 2)) return (int)cudaErrorInvalidValue;
    dim3 grid(T, kv_heads);
    ps::dfl_ring_attention_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kb, (const __nv_bfloat16*)vb, ldkv,
                                                            (const __nv_bfloat16*)k_ring, (const __nv_bfloat16*)v_ring, (const int*)ring_pos,
                                                            (const int*)pos, T, window, q_heads, kv_heads, scale, (__nv_bfloat16*)out, ldo);
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
    ps::dfl_select_kernel<<<1, 128, 0, stream>>>((const int*)top_ids, (const float*)top_logits, kk, (const float*)hproj, rank,
                                                 (const __nv_bfloat16*)pred_cb, (const __nv_bfloat16*)succ_cb, (const int*)anchor_dev,
                                                 anchor_value, K, vocab, (int*)out_tokens);
    return PS_LAUNCH_CHECK();
}
