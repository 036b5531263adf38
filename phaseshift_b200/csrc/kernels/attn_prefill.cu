// Causal paged attention for prefill-sized steps: one CTA = 64 consecutive query rows of one sequence
// and one query head, streaming 64-token K/V tiles from the paged pools through shared memory, with
// both products (Q K^T and P V) on the tensor cores (bf16 mma.sync m16n8k16, fp32 accumulation) and the
// online softmax kept in the accumulator registers, flash-attention style.  The probabilities never
// leave registers: the Q K^T accumulator fragments are re-packed as the A operand of the P V product.
// FP8 pools widen exactly to bf16 when a tile is staged; the per-token K scale multiplies the scores
// and the per-token V scale multiplies the probabilities, as in the decode kernel.  The epilogue applies
// the sigmoid output gate and writes bf16, so o_proj reads its input directly.
//
// The reference's prefill attention (src/phaseshift/models/qwen35/kernels/optimized/attention/
// paged_prefill.hip) tiles 16 query rows per wave with WMMA; here a warp owns 16 rows and a CTA 64, and
// the six query heads that share a KV head run as neighbouring CTAs so their K/V tiles hit in L2.
// Decode and speculative verification stay on the split-KV kernel (paged_attention.cu), whose per-row
// arithmetic does not depend on the batch.
#include "ps_common.cuh"

namespace ps {

constexpr int kPfRows = 64;      // query rows per CTA
constexpr int kPfTok = 64;       // tokens per K/V tile
constexpr int kPfThreads = 128;

struct AttnPrefillArgs {
    const __nv_bfloat16* q;      // [rows, Hq, D]
    const void* k_pool; const void* v_pool; const float* k_scale; const float* v_scale;
    const int* block_table; int max_blocks; int page_tokens; int num_pages;
    const int* seqs;             // [n_seqs][4] = row_start, n_rows, slot, pos_start
    int Hq, Hkv; float scale_log2; int kv_fp8; int min_rows;
    const __nv_bfloat16* gate; int ld_gate; int gate_head_stride; int gate_offset;
    __nv_bfloat16* out;          // [rows, Hq*D]
    uint32_t* status;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Stage 64 tokens [t0, t0+64) of one kv head into shared memory as bf16 rows of pitch D+8 (tokens at
// or beyond `end` become zero rows).
template <int D>
__device__ __forceinline__ void stage_tile(const AttnPrefillArgs& a, const void* pool, const float* scale_pool,
                                           __nv_bfloat16* dst, float* sdst, int slot, int kvh, int t0, int end, bool& bad) {
    constexpr int P = D + 8;
    if (!a.kv_fp8) {
        constexpr int PPR = D / 8;               // 16-byte pieces per token row
        for (int p = threadIdx.x; p < kPfTok * PPR; p += kPfThreads) {
            const int t = p / PPR, c = p % PPR, tok = t0 + t;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok < end) {
                const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
                if (page < 0 || page >= a.num_pages) bad = true;
                else v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(pool) +
                               (((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens) * D) + c);
            }
            *reinterpret_cast<uint4*>(dst + t * P + c * 8) = v;
        }
    } else {
        constexpr int PPR = D / 16;
        for (int p = threadIdx.x; p < kPfTok * PPR; p += kPfThreads) {
            const int t = p / PPR, c = p % PPR, tok = t0 + t;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok < end) {
                const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
                if (page < 0 || page >= a.num_pages) bad = true;
                else v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(pool) +
                               (((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens) * D) + c);
            }
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float lo = e4m3_to_f32((w[j >> 1] >> ((j & 1) * 16)) & 0xff);
                const float hi = e4m3_to_f32((w[j >> 1] >> ((j & 1) * 16 + 8)) & 0xff);
                o[j] = f32x2_to_bf16x2_bits(lo, hi);
            }
            *reinterpret_cast<uint4*>(dst + t * P + c * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + t * P + c * 16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        if (threadIdx.x < kPfTok) {
            const int tok = t0 + threadIdx.x;
            float s = 1.f;
            if (tok < end) {
                const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
                if (page >= 0 && page < a.num_pages)
                    s = scale_pool[((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens];
            }
            sdst[threadIdx.x] = s;
        }
    }
}

// grid = (q tiles, Hq, n_seqs); the heaviest (latest) query tiles are scheduled first.
template <int D>
__global__ void __launch_bounds__(kPfThreads) attn_prefill_kernel(const AttnPrefillArgs a) {
    constexpr int P = D + 8;
    extern __shared__ __align__(16) unsigned char smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* sK = sQ + kPfRows * P;
    __nv_bfloat16* sV = sK + kPfTok * P;
    float* sKs = reinterpret_cast<float*>(sV + kPfTok * P);
    float* sVs = sKs + kPfTok;

    const int* sd = a.seqs + 4 * blockIdx.z;
    const int row_start = sd[0], n_rows = sd[1], slot = sd[2], pos_start = sd[3];
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int r_begin = tile * kPfRows;
    if (r_begin >= n_rows || slot < 0 || n_rows <= a.min_rows) return;
    const int nq = min(kPfRows, n_rows - r_begin);
    const int h = blockIdx.y, G = a.Hq / a.Hkv, kvh = h / G;
    const int pos_q0 = pos_start + r_begin;
    const int kv_end = pos_q0 + nq;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

    for (int p = t; p < kPfRows * (D / 8); p += kPfThreads) {
        const int r = p / (D / 8), c = p % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = __ldg(reinterpret_cast<const uint4*>(a.q + ((size_t)(row_start + r_begin + r) * a.Hq + h) * D) + c);
        *reinterpret_cast<uint4*>(sQ + r * P + c * 8) = v;
    }
    if (t < kPfTok) { sKs[t] = 1.f; sVs[t] = 1.f; }

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-1.0e30f, -1.0e30f}, l_run[2] = {0.f, 0.f};
    const int rpos0 = pos_q0 + warp * 16 + (lane >> 2);       // position of this thread's first row (second = +8)
    bool bad = false;

    for (int t0 = 0; t0 < kv_end; t0 += kPfTok) {
        __syncthreads();                                        // previous tile consumed (and Q staged)
        stage_tile<D>(a, a.k_pool, a.k_scale, sK, sKs, slot, kvh, t0, kv_end, bad);
        stage_tile<D>(a, a.v_pool, a.v_scale, sV, sVs, slot, kvh, t0, kv_end, bad);
        __syncthreads();
        // rows of this warp that see nothing in this tile can skip the whole tile
        if (t0 > pos_q0 + warp * 16 + 15) continue;

        // ---- S = Q K^T : 16 rows x 64 tokens per warp
        float s[kPfTok / 8][4];
#pragma unroll
        for (int j = 0; j < kPfTok / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll 4
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t af[4];
            ldsm_x4(af, sQ + (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int n2 = 0; n2 < kPfTok / 16; ++n2) {
                uint32_t bf[4];
                ldsm_x4(bf, sK + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * P + kk * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(s[2 * n2], af, bf[0], bf[1]);
                mma_bf16_16816(s[2 * n2 + 1], af, bf[2], bf[3]);
            }
        }
        // ---- scale, causal mask, online softmax (rows lane/4 and lane/4 + 8)
        float mx[2] = {-1.0e30f, -1.0e30f};
#pragma unroll
        for (int j = 0; j < kPfTok / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int tl = 8 * j + (lane & 3) * 2 + (e & 1);
                const int tok = t0 + tl;
                const int rp = rpos0 + (e >> 1) * 8;
                float v = s[j][e] * a.scale_log2 * sKs[tl];
                if (tok > rp) v = -1.0e30f;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            alpha[r] = exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= alpha[r];
        }
        uint32_t pf[kPfTok / 16][4];
#pragma unroll
        for (int j = 0; j < kPfTok / 8; ++j) {
            const int tl = 8 * j + (lane & 3) * 2;
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = s[j][e] > -0.5e30f ? exp2f(s[j][e] - m_run[e >> 1]) : 0.f;
                l_run[e >> 1] += p[e];
            }
            const float v0 = sVs[tl], v1 = sVs[tl + 1];
            pf[j >> 1][(j & 1) * 2 + 0] = f32x2_to_bf16x2_bits(p[0] * v0, p[1] * v1);
            pf[j >> 1][(j & 1) * 2 + 1] = f32x2_to_bf16x2_bits(p[2] * v0, p[3] * v1);
        }
#pragma unroll
        for (int j = 0; j < D / 8; ++j) { o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1]; }
        // ---- O += P V : k = tokens, n = dims
#pragma unroll
        for (int kk = 0; kk < kPfTok / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t bf[4];
                ldsm_x4_t(bf, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P + n2 * 16 + (lane >> 4) * 8);
                mma_bf16_16816(o[2 * n2], pf[kk], bf[0], bf[1]);
                mma_bf16_16816(o[2 * n2 + 1], pf[kk], bf[2], bf[3]);
            }
        }
    }
    if (bad) set_status(a.status, PS_DEV_BAD_INDEX);
    // ---- epilogue: normalise, gate, store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = warp * 16 + (lane >> 2) + r * 8;
        if (lr >= nq) continue;
        const size_t row = (size_t)(row_start + r_begin + lr);
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            const int d = 8 * j + (lane & 3) * 2;
            float v0 = bf16_to_f32(f32_to_bf16(o[j][2 * r] * inv)), v1 = bf16_to_f32(f32_to_bf16(o[j][2 * r + 1] * inv));
            if (a.gate != nullptr) {
                const float2 gv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(
                    a.gate + row * a.ld_gate + (size_t)h * a.gate_head_stride + a.gate_offset + d));
                v0 *= sigmoid_f(gv.x); v1 *= sigmoid_f(gv.y);
            }
            *reinterpret_cast<uint32_t*>(a.out + (row * a.Hq + h) * D + d) = f32x2_to_bf16x2_bits(v0, v1);
        }
    }
}

// ---- bf16 pools: the same tile loop with K/V tiles copied asynchronously (cp.async, 16 bytes per request):
// the K tile of step t+1 is in flight while step t does its softmax and P V, the V tile of step t+1 while
// step t+1 computes Q K^T, so the tensor cores no longer wait for a full global -> shared round trip per tile.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;                 // src-size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__device__ __forceinline__ void issue_tile(const AttnPrefillArgs& a, const void* pool, __nv_bfloat16* dst, int slot, int kvh, int t0,
                                           int end, bool& bad) {
    constexpr int P = D + 8, PPR = D / 8;
    if (t0 < end) {
        for (int p = threadIdx.x; p < kPfTok * PPR; p += kPfThreads) {
            const int t = p / PPR, c = p % PPR, tok = t0 + t;
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(pool);
            bool ok = tok < end;
            if (ok) {
                const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
                if (page < 0 || page >= a.num_pages) { bad = true; ok = false; }
                else src += (((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens) * D + c * 8;
            }
            cp_async16(dst + t * P + c * 8, src, ok);
        }
    }
    cp_async_commit();                              // always commit so the group count stays uniform
}

template <int D>
__global__ void __launch_bounds__(kPfThreads) attn_prefill_async_kernel(const AttnPrefillArgs a) {
    constexpr int P = D + 8;
    extern __shared__ __align__(16) unsigned char smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* sK = sQ + kPfRows * P;
    __nv_bfloat16* sV = sK + kPfTok * P;

    const int* sd = a.seqs + 4 * blockIdx.z;
    const int row_start = sd[0], n_rows = sd[1], slot = sd[2], pos_start = sd[3];
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int r_begin = tile * kPfRows;
    if (r_begin >= n_rows || slot < 0 || n_rows <= a.min_rows) return;
    const int nq = min(kPfRows, n_rows - r_begin);
    const int h = blockIdx.y, G = a.Hq / a.Hkv, kvh = h / G;
    const int pos_q0 = pos_start + r_begin;
    const int kv_end = pos_q0 + nq;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    bool bad = false;

    issue_tile<D>(a, a.k_pool, sK, slot, kvh, 0, kv_end, bad);
    issue_tile<D>(a, a.v_pool, sV, slot, kvh, 0, kv_end, bad);
    for (int p = t; p < kPfRows * (D / 8); p += kPfThreads) {
        const int r = p / (D / 8), c = p % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = __ldg(reinterpret_cast<const uint4*>(a.q + ((size_t)(row_start + r_begin + r) * a.Hq + h) * D) + c);
        *reinterpret_cast<uint4*>(sQ + r * P + c * 8) = v;
    }

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-1.0e30f, -1.0e30f}, l_run[2] = {0.f, 0.f};
    const int rpos0 = pos_q0 + warp * 16 + (lane >> 2);

    for (int t0 = 0; t0 < kv_end; t0 += kPfTok) {
        const bool live = t0 <= pos_q0 + warp * 16 + 15;       // some row of this warp sees this tile
        cp_async_wait<1>();                                     // K(t) has landed (V(t) may still be in flight)
        __syncthreads();
        float s[kPfTok / 8][4];
#pragma unroll
        for (int j = 0; j < kPfTok / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
        if (live) {
#pragma unroll 4
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t af[4];
                ldsm_x4(af, sQ + (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int n2 = 0; n2 < kPfTok / 16; ++n2) {
                    uint32_t bf[4];
                    ldsm_x4(bf, sK + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * P + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16_16816(s[2 * n2], af, bf[0], bf[1]);
                    mma_bf16_16816(s[2 * n2 + 1], af, bf[2], bf[3]);
                }
            }
        }
        __syncthreads();                                        // every warp is done with the K tile
        issue_tile<D>(a, a.k_pool, sK, slot, kvh, t0 + kPfTok, kv_end, bad);
        uint32_t pf[kPfTok / 16][4];
        float alpha[2] = {1.f, 1.f};
        if (live) {
            float mx[2] = {-1.0e30f, -1.0e30f};
#pragma unroll
            for (int j = 0; j < kPfTok / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int tok = t0 + 8 * j + (lane & 3) * 2 + (e & 1);
                    float v = s[j][e] * a.scale_log2;
                    if (tok > rpos0 + (e >> 1) * 8) v = -1.0e30f;
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                alpha[r] = exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
                l_run[r] *= alpha[r];
            }
#pragma unroll
            for (int j = 0; j < kPfTok / 8; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[e] = s[j][e] > -0.5e30f ? exp2f(s[j][e] - m_run[e >> 1]) : 0.f;
                    l_run[e >> 1] += p[e];
                }
                pf[j >> 1][(j & 1) * 2 + 0] = f32x2_to_bf16x2_bits(p[0], p[1]);
                pf[j >> 1][(j & 1) * 2 + 1] = f32x2_to_bf16x2_bits(p[2], p[3]);
            }
#pragma unroll
            for (int j = 0; j < D / 8; ++j) { o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1]; }
        }
        cp_async_wait<1>();                                     // V(t) has landed (K(t+1) may still be in flight)
        __syncthreads();
        if (live) {
#pragma unroll
            for (int kk = 0; kk < kPfTok / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < D / 16; ++n2) {
                    uint32_t bf[4];
                    ldsm_x4_t(bf, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P + n2 * 16 + (lane >> 4) * 8);
                    mma_bf16_16816(o[2 * n2], pf[kk], bf[0], bf[1]);
                    mma_bf16_16816(o[2 * n2 + 1], pf[kk], bf[2], bf[3]);
                }
            }
        }
        __syncthreads();                                        // every warp is done with the V tile
        issue_tile<D>(a, a.v_pool, sV, slot, kvh, t0 + kPfTok, kv_end, bad);
    }
    cp_async_wait<0>();
    if (bad) set_status(a.status, PS_DEV_BAD_INDEX);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = warp * 16 + (lane >> 2) + r * 8;
        if (lr >= nq) continue;
        const size_t row = (size_t)(row_start + r_begin + lr);
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            const int d = 8 * j + (lane & 3) * 2;
            float v0 = bf16_to_f32(f32_to_bf16(o[j][2 * r] * inv)), v1 = bf16_to_f32(f32_to_bf16(o[j][2 * r + 1] * inv));
            if (a.gate != nullptr) {
                const float2 gv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(
                    a.gate + row * a.ld_gate + (size_t)h * a.gate_head_stride + a.gate_offset + d));
                v0 *= sigmoid_f(gv.x); v1 *= sigmoid_f(gv.y);
            }
            *reinterpret_cast<uint32_t*>(a.out + (row * a.Hq + h) * D + d) = f32x2_to_bf16x2_bits(v0, v1);
        }
    }
}

template <int D>
static int launch_prefill(const AttnPrefillArgs& a, int max_q_tiles, int n_seqs, cudaStream_t stream) {
    const size_t smem = (size_t)(kPfRows + 2 * kPfTok) * (D + 8) * 2 + 2 * kPfTok * sizeof(float);
    static bool set = false;
    if (!set) {
        cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(attn_prefill_async_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        set = true;
    }
    if (a.kv_fp8) attn_prefill_kernel<D><<<dim3(max_q_tiles, a.Hq, n_seqs), kPfThreads, smem, stream>>>(a);
    else attn_prefill_async_kernel<D><<<dim3(max_q_tiles, a.Hq, n_seqs), kPfThreads, smem, stream>>>(a);
    return PS_LAUNCH_CHECK();
}

// attn_prefill_tc.cu: the tcgen05 kernel for head dim 256 and pages of 16 / 32 / 64 tokens (FP8 pools through a bf16 scratch pool)
bool attn_prefill_tc_supported(int D, int page_tokens, int kv_fp8, const void* q, const void* k_pool, const void* v_pool,
                               const void* gate, int ld_gate, int gate_head_stride, int gate_offset, const void* deq_k);
int launch_attn_prefill_tc(const void* q, int q_rows, const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale,
                           int kv_fp8, const void* block_table, int max_blocks, int num_pages, int page_tokens, const void* seqs,
                           int n_seqs, int max_seq_rows, int min_rows, int Hq, int Hkv, float sm_scale, const void* gate, int ld_gate,
                           int gate_head_stride, int gate_offset, void* deq_k, void* deq_v, int deq_pages, void* deq_bt, void* deq_seqs,
                           void* out, void* status, cudaStream_t stream);

}  // namespace ps

// `max_seq_rows`: upper bound of n_rows over the step's sequences (sizes the grid); `q_rows`: rows of the q tensor;
// `min_rows`: sequences with at most this many rows are skipped (the caller runs the split-KV kernel on their rows);
// `deq_*`: optional bf16 scratch pool ([deq_pages, Hkv, page_tokens, D] twice), block table [n_seqs, max_blocks] and
// sequence descriptors [n_seqs, 4] that let FP8 pools take the tensor-core kernel.
PS_API int ps_attn_prefill(const void* q, const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale,
                           const void* block_table, int max_blocks, int page_tokens, int num_pages, const void* seqs,
                           int n_seqs, int max_seq_rows, int q_rows, int min_rows, int Hq, int Hkv, int D, float sm_scale, int kv_fp8,
                           const void* gate, int ld_gate, int gate_head_stride, int gate_offset, void* deq_k, void* deq_v,
                           int deq_pages, void* deq_bt, void* deq_seqs, void* out, void* status, cudaStream_t stream) {
    using namespace ps;
    if (n_seqs <= 0 || max_seq_rows <= 0 || Hkv <= 0 || (Hq % Hkv) || q_rows < max_seq_rows) return (int)cudaErrorInvalidValue;
    if (attn_prefill_tc_supported(D, page_tokens, kv_fp8, q, k_pool, v_pool, gate, ld_gate, gate_head_stride, gate_offset, deq_k))
        return launch_attn_prefill_tc(q, q_rows, k_pool, v_pool, k_scale, v_scale, kv_fp8, block_table, max_blocks, num_pages, page_tokens,
                                      seqs, n_seqs, max_seq_rows, min_rows, Hq, Hkv, sm_scale, gate, ld_gate, gate_head_stride, gate_offset,
                                      deq_k, deq_v, deq_pages, deq_bt, deq_seqs, out, status, stream);
    AttnPrefillArgs a;
    a.q = (const __nv_bfloat16*)q; a.k_pool = k_pool; a.v_pool = v_pool; a.k_scale = (const float*)k_scale;
    a.v_scale = (const float*)v_scale; a.block_table = (const int*)block_table; a.max_blocks = max_blocks;
    a.page_tokens = page_tokens; a.num_pages = num_pages; a.seqs = (const int*)seqs; a.Hq = Hq; a.Hkv = Hkv;
    a.scale_log2 = sm_scale * 1.4426950408889634f; a.kv_fp8 = kv_fp8; a.gate = (const __nv_bfloat16*)gate;
    a.ld_gate = ld_gate; a.gate_head_stride = gate_head_stride; a.gate_offset = gate_offset;
    a.out = (__nv_bfloat16*)out; a.status = (uint32_t*)status; a.min_rows = min_rows;
    const int tiles = (max_seq_rows + kPfRows - 1) / kPfRows;
    if (D == 256) return launch_prefill<256>(a, tiles, n_seqs, stream);
    if (D == 128) return launch_prefill<128>(a, tiles, n_seqs, stream);
    if (D == 64) return launch_prefill<64>(a, tiles, n_seqs, stream);
    return (int)cudaErrorInvalidValue;
}
