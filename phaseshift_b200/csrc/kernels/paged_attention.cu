// Paged causal attention over BF16 / FP8-E4M3 KV pages: split-KV partial pass + merge pass.
//
// Flash-decoding structure like the reference's split-KV path (src/phaseshift/models/qwen35/kernels/
// optimized/attention/paged_decode.hip:264-300,743-780; plan in runtime/paged_attention_dispatch.hip:
// 437-468), with two differences that matter on B200:
//   * the split length is a fixed number of tokens chosen once per engine, never a function of the
//     batch, so a row's result is bit-identical whether it is decoded alone, verified among 16
//     speculative rows or batched with other requests (the reference gets this by forcing S=16);
//   * the merge pass also applies the sigmoid output gate, so o_proj reads its input directly.
// One CTA = (split, kv head, row) and serves all G = Hq/Hkv query heads that share the K/V tile.
//
// K/V pools: [num_pages, Hkv, page_tokens, D]; FP8 pools carry one f32 scale per (page, head, token).
#include <stdio.h>

#include "ps_common.cuh"
#include "ps_noalloc.h"

namespace ps {

constexpr int kAttnTile = 32;      // tokens per shared-memory tile
constexpr int kAttnThreads = 256;
constexpr int kAttnMaxG = 8;
constexpr int kAttnMaxD = 256;

struct PagedAttnArgs {
    const __nv_bfloat16* q;      // [rows, Hq, D]
    const void* k_pool; const void* v_pool; const float* k_scale; const float* v_scale;
    const int* block_table; int max_blocks; int page_tokens; int num_pages;
    const int* row_slot; const int* row_pos;
    int rows, Hq, Hkv, D; float sm_scale; int kv_fp8;
    int split_tokens, max_splits;
    float* part_acc;   // [rows, Hq, max_splits, D]
    float* part_ml;    // [rows, Hq, max_splits, 2]  (running max, running sum)
    uint32_t* status;
};

struct TileRegs { uint4 k[4]; uint4 v[4]; float ks, vs; };

// Fetch one 32-token tile (K and V rows of this kv head) into registers.  Thread t covers 16-byte
// pieces t, t+256, ... of the [32, D] tile; threads 0..31 also fetch the fp8 token scales.
__device__ __forceinline__ void tile_fetch(const PagedAttnArgs& a, TileRegs& r, int slot, int kvh, int tok0,
                                           int visible, bool& bad) {
    const int esz = a.kv_fp8 ? 1 : 2;
    const int row_bytes = a.D * esz;
    const int pieces_per_row = row_bytes / 16;
    const int total = kAttnTile * pieces_per_row;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = threadIdx.x + i * kAttnThreads;
        r.k[i] = make_uint4(0, 0, 0, 0); r.v[i] = make_uint4(0, 0, 0, 0);
        if (p < total) {
            const int t = p / pieces_per_row, c = p % pieces_per_row;
            const int tok = tok0 + t;
            if (tok < visible) {
                const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
                if (page < 0 || page >= a.num_pages) { bad = true; continue; }
                const size_t off = (((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens) * row_bytes + c * 16;
                r.k[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.k_pool) + off));
                r.v[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.v_pool) + off));
            }
        }
    }
    r.ks = 1.f; r.vs = 1.f;
    if (a.kv_fp8 && threadIdx.x < kAttnTile) {
        const int tok = tok0 + threadIdx.x;
        if (tok < visible) {
            const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
            if (page >= 0 && page < a.num_pages) {
                const size_t so = ((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens;
                r.ks = a.k_scale[so]; r.vs = a.v_scale[so];
            }
        }
    }
}

// Two E4M3 codes (low byte first) -> two bf16 values (exact: three mantissa bits): one hardware conversion to f16x2, then
// through fp32.  NaN codes stay NaN.
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint16_t two) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(two));
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    return f32x2_to_bf16x2_bits(f.x, f.y);
}

// Registers -> shared memory as bf16 (fp8 codes widen exactly).  K rows are padded by 8 elements.
__device__ __forceinline__ void tile_store(const PagedAttnArgs& a, const TileRegs& r, __nv_bfloat16* ks,
                                           __nv_bfloat16* vs, float* kscale, float* vscale) {
    const int kpitch = a.D + 8;
    if (!a.kv_fp8) {
        const int ppr = a.D * 2 / 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = threadIdx.x + i * kAttnThreads;
            if (p < kAttnTile * ppr) {
                const int t = p / ppr, c = p % ppr;
                *reinterpret_cast<uint4*>(ks + t * kpitch + c * 8) = r.k[i];
                *reinterpret_cast<uint4*>(vs + t * a.D + c * 8) = r.v[i];
            }
        }
    } else {
        const int ppr = a.D / 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = threadIdx.x + i * kAttnThreads;
            if (p < kAttnTile * ppr) {
                const int t = p / ppr, c = p % ppr;
                const uint32_t kw[4] = {r.k[i].x, r.k[i].y, r.k[i].z, r.k[i].w};
                const uint32_t vw[4] = {r.v[i].x, r.v[i].y, r.v[i].z, r.v[i].w};
                // two codes per conversion instruction, sixteen values leave as two 16-byte stores per matrix
                uint32_t ko[8], vo[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    ko[j] = e4m3x2_to_bf16x2((uint16_t)(kw[j >> 1] >> ((j & 1) * 16)));
                    vo[j] = e4m3x2_to_bf16x2((uint16_t)(vw[j >> 1] >> ((j & 1) * 16)));
                }
                uint4* kd = reinterpret_cast<uint4*>(ks + t * kpitch + c * 16);
                uint4* vd = reinterpret_cast<uint4*>(vs + t * a.D + c * 16);
                kd[0] = make_uint4(ko[0], ko[1], ko[2], ko[3]); kd[1] = make_uint4(ko[4], ko[5], ko[6], ko[7]);
                vd[0] = make_uint4(vo[0], vo[1], vo[2], vo[3]); vd[1] = make_uint4(vo[4], vo[5], vo[6], vo[7]);
            }
        }
        if (threadIdx.x < kAttnTile) { kscale[threadIdx.x] = r.ks; vscale[threadIdx.x] = r.vs; }
    }
}

__global__ void __launch_bounds__(kAttnThreads) paged_attn_split_kernel(const PagedAttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int D = a.D, G = a.Hq / a.Hkv, kpitch = D + 8;
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem);            // [32][D+8]
    __nv_bfloat16* vs = ks + kAttnTile * kpitch;                           // [32][D]
    float* qs = reinterpret_cast<float*>(vs + kAttnTile * D);              // [G][D]
    float* ps_ = qs + kAttnMaxG * D;                                       // [G][32]
    float* alpha = ps_ + kAttnMaxG * kAttnTile;                            // [G]
    float* kscale = alpha + kAttnMaxG;                                     // [32]
    float* vscale = kscale + kAttnTile;                                    // [32]

    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();
    const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int visible = a.row_pos[row] + 1;
    const int tok_begin = split * a.split_tokens;
    if (tok_begin >= visible) return;
    const int tok_end = min(visible, tok_begin + a.split_tokens);
    const int slot = a.row_slot[row];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

    for (int i = t; i < G * D; i += kAttnThreads) {
        const int g = i / D, d = i % D;
        qs[i] = bf16_to_f32(a.q[((size_t)row * a.Hq + kvh * G + g) * D + d]) * a.sm_scale;
    }
    if (t < kAttnTile) { kscale[t] = 1.f; vscale[t] = 1.f; }
    float acc[kAttnMaxG];
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) acc[g] = 0.f;
    float m_run = -3.0e38f, l_run = 0.f;   // owned by warp g (all lanes hold the same value)

    bool bad = false;
    TileRegs regs;
    tile_fetch(a, regs, slot, kvh, tok_begin, tok_end, bad);
    for (int tok0 = tok_begin; tok0 < tok_end; tok0 += kAttnTile) {
        __syncthreads();                       // previous tile fully consumed
        tile_store(a, regs, ks, vs, kscale, vscale);
        __syncthreads();
        if (tok0 + kAttnTile < tok_end) tile_fetch(a, regs, slot, kvh, tok0 + kAttnTile, tok_end, bad);

        // scores: warp g, lane = token
        if (warp < G) {
            const int tok = tok0 + lane;
            float s = 0.f;
            const __nv_bfloat16* kr = ks + lane * kpitch;
            const float* qg = qs + warp * D;
            for (int d = 0; d < D; d += 8) {
                const uint4 kk = *reinterpret_cast<const uint4*>(kr + d);
                const float4 qa = *reinterpret_cast<const float4*>(qg + d);
                const float4 qb = *reinterpret_cast<const float4*>(qg + d + 4);
                const float2 k0 = bf16x2_bits_to_f32x2(kk.x), k1 = bf16x2_bits_to_f32x2(kk.y);
                const float2 k2 = bf16x2_bits_to_f32x2(kk.z), k3 = bf16x2_bits_to_f32x2(kk.w);
                s = fmaf(k0.x, qa.x, s); s = fmaf(k0.y, qa.y, s); s = fmaf(k1.x, qa.z, s); s = fmaf(k1.y, qa.w, s);
                s = fmaf(k2.x, qb.x, s); s = fmaf(k2.y, qb.y, s); s = fmaf(k3.x, qb.z, s); s = fmaf(k3.y, qb.w, s);
            }
            s *= kscale[lane];
            const bool live = tok < tok_end;
            if (!live) s = -3.0e38f;
            const float m_new = fmaxf(m_run, warp_max(s));
            const float p = live ? __expf(s - m_new) : 0.f;
            const float al = __expf(m_run - m_new);
            l_run = l_run * al + warp_sum(p);
            m_run = m_new;
            ps_[warp * kAttnTile + lane] = p * vscale[lane];
            if (lane == 0) alpha[warp] = al;
        }
        __syncthreads();
        // PV: thread = output dim, all heads
        if (t < D) {
            // tokens outermost, four at a time: a value of V is read once for all heads and the heads' probabilities come
            // as one broadcast 16-byte load each (the loop used to issue two shared-memory loads per multiply-add, which
            // bounded batched decode); per head the additions still run in token order, so the result is unchanged
#pragma unroll
            for (int g = 0; g < kAttnMaxG; ++g)
                if (g < G) acc[g] *= alpha[g];
#pragma unroll 2
            for (int j0 = 0; j0 < kAttnTile; j0 += 4) {
                float vv[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) vv[jj] = bf16_to_f32(vs[(j0 + jj) * D + t]);
#pragma unroll
                for (int g = 0; g < kAttnMaxG; ++g) {
                    if (g < G) {
                        const float4 pq = *reinterpret_cast<const float4*>(ps_ + g * kAttnTile + j0);
                        float s = acc[g];
                        s = fmaf(pq.x, vv[0], s); s = fmaf(pq.y, vv[1], s); s = fmaf(pq.z, vv[2], s); s = fmaf(pq.w, vv[3], s);
                        acc[g] = s;
                    }
                }
            }
        }
    }
    if (bad && t == 0) set_status(a.status, PS_DEV_BAD_INDEX);
    // write partials
    if (t < D) {
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g)
            if (g < G) a.part_acc[(((size_t)row * a.Hq + kvh * G + g) * a.max_splits + split) * D + t] = acc[g];
    }
    if (warp < G && lane == 0) {
        float* ml = a.part_ml + (((size_t)row * a.Hq + kvh * G + warp) * a.max_splits + split) * 2;
        ml[0] = m_run; ml[1] = l_run;
    }
}

struct AttnMergeArgs {
    const float* part_acc; const float* part_ml; const int* row_pos;
    int rows, Hq, D, split_tokens, max_splits;
    const __nv_bfloat16* gate; int ld_gate; int gate_head_stride; int gate_offset;   // optional sigmoid gate
    __nv_bfloat16* out;   // [rows, Hq*D]
};

// grid = (Hq, rows), block = D threads.  The split weights exp(m_s - max m) are computed once, in
// parallel (thread s owns split s), then every thread adds its output dimension over the splits in
// ascending order, so the result depends only on the row's position, never on the batch.
constexpr int kAttnMaxSplits = 1024;
__global__ void paged_attn_merge_kernel(const AttnMergeArgs a) {
    __shared__ float s_w[kAttnMaxSplits];
    __shared__ float s_red[64];
    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();
    const int h = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
    const int visible = a.row_pos[row] + 1;
    if (visible < 0) return;                                            // position -2: a row another kernel of the step owns
    const int n = (visible + a.split_tokens - 1) / a.split_tokens;      // 0 for a padding row
    const float* ml = a.part_ml + ((size_t)row * a.Hq + h) * a.max_splits * 2;
    const float* pa = a.part_acc + ((size_t)row * a.Hq + h) * a.max_splits * a.D;
    float m = -3.0e38f;
    for (int s = d; s < n; s += blockDim.x) m = fmaxf(m, ml[2 * s]);
    m = block_max(m, s_red);
    float l = 0.f;
    for (int s = d; s < n; s += blockDim.x) {
        const float w = __expf(ml[2 * s] - m);
        s_w[s] = w;
        l = fmaf(w, ml[2 * s + 1], l);
    }
    l = block_sum(l, s_red + 32);      // its barriers also publish s_w
    float o = 0.f;
#pragma unroll 4
    for (int s = 0; s < n; ++s) o = fmaf(s_w[s], pa[(size_t)s * a.D + d], o);
    float v = l > 0.f ? o / l : 0.f;
    if (a.gate != nullptr) {
        v = bf16_to_f32(f32_to_bf16(v));
        const float g = bf16_to_f32(a.gate[(size_t)row * a.ld_gate + h * a.gate_head_stride + a.gate_offset + d]);
        v *= sigmoid_f(g);
    }
    a.out[((size_t)row * a.Hq + h) * a.D + d] = f32_to_bf16(v);
}

}  // namespace ps

PS_API int ps_paged_attention(const void* q, const void* k_pool, const void* v_pool, const void* k_scale,
                              const void* v_scale, const void* block_table, int max_blocks, int page_tokens,
                              int num_pages, const void* row_slot, const void* row_pos, int rows, int Hq, int Hkv,
                              int D, float sm_scale, int kv_fp8, int split_tokens, int max_splits, int max_visible,
                              void* part_acc, void* part_ml, const void* gate, int ld_gate, int gate_head_stride,
                              int gate_offset, void* out, void* status, cudaStream_t stream) {
    using namespace ps;
    const int G = Hkv > 0 ? Hq / Hkv : 0;
    if (G < 1 || G > kAttnMaxG || D > kAttnMaxD || (D % 32) || (split_tokens % kAttnTile) || rows <= 0)
        return (int)cudaErrorInvalidValue;
    PagedAttnArgs a;
    a.q = (const __nv_bfloat16*)q; a.k_pool = k_pool; a.v_pool = v_pool; a.k_scale = (const float*)k_scale;
    a.v_scale = (const float*)v_scale; a.block_table = (const int*)block_table; a.max_blocks = max_blocks;
    a.page_tokens = page_tokens; a.num_pages = num_pages; a.row_slot = (const int*)row_slot;
    a.row_pos = (const int*)row_pos; a.rows = rows; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.sm_scale = sm_scale;
    a.kv_fp8 = kv_fp8; a.split_tokens = split_tokens; a.max_splits = max_splits;
    a.part_acc = (float*)part_acc; a.part_ml = (float*)part_ml; a.status = (uint32_t*)status;
    int n_splits = (max_visible + split_tokens - 1) / split_tokens;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > max_splits || max_splits > kAttnMaxSplits) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)kAttnTile * (D + 8) * 2 + (size_t)kAttnTile * D * 2 +
                        sizeof(float) * (kAttnMaxG * D + kAttnMaxG * kAttnTile + kAttnMaxG + 2 * kAttnTile);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(paged_attn_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        attr_set = true;
    }
    dim3 grid(n_splits, Hkv, rows);
    int err = launch_pdl(paged_attn_split_kernel, grid, dim3(kAttnThreads), smem, stream, a);
    if (err) return err;
    AttnMergeArgs m;
    m.part_acc = a.part_acc; m.part_ml = a.part_ml; m.row_pos = a.row_pos; m.rows = rows; m.Hq = Hq; m.D = D;
    m.split_tokens = split_tokens; m.max_splits = max_splits; m.gate = (const __nv_bfloat16*)gate;
    m.ld_gate = ld_gate; m.gate_head_stride = gate_head_stride; m.gate_offset = gate_offset;
    m.out = (__nv_bfloat16*)out;
    return launch_pdl(paged_attn_merge_kernel, dim3(Hq, rows), dim3(D), 0, stream, m);
}

// The merge pass alone: for partials produced by another split-KV kernel (attn_prefill_tc.cu's decode variant) in the same
// layout.  Same arguments as the tail of ps_paged_attention.
PS_API int ps_paged_attention_merge(const void* part_acc, const void* part_ml, const void* row_pos, int rows, int Hq, int D,
                                    int split_tokens, int max_splits, const void* gate, int ld_gate, int gate_head_stride,
                                    int gate_offset, void* out, cudaStream_t stream) {
    using namespace ps;
    if (rows <= 0 || Hq <= 0 || D <= 0 || D > kAttnMaxD || max_splits > kAttnMaxSplits) return (int)cudaErrorInvalidValue;
    AttnMergeArgs m;
    m.part_acc = (const float*)part_acc; m.part_ml = (const float*)part_ml; m.row_pos = (const int*)row_pos; m.rows = rows; m.Hq = Hq; m.D = D;
    m.split_tokens = split_tokens; m.max_splits = max_splits; m.gate = (const __nv_bfloat16*)gate;
    m.ld_gate = ld_gate; m.gate_head_stride = gate_head_stride; m.gate_offset = gate_offset;
    m.out = (__nv_bfloat16*)out;
    return launch_pdl(paged_attn_merge_kernel, dim3(Hq, rows), dim3(D), 0, stream, m);
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant: identical kernels, partial results in static device storage (ps_noalloc.h).
namespace ps {
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static void* g_noalloc_ptr[64] = {nullptr};           // device address of the array, per device ordinal
static thread_local char g_noalloc_err[256] = "";
}  // namespace ps

PS_API const char* ps_noalloc_last_error(void) { return ps::g_noalloc_err; }

PS_API int ps_paged_attention_noalloc(const void* q, const void* k_pool, const void* v_pool, const void* k_scale,
                                      const void* v_scale, const void* block_table, int max_blocks, int page_tokens,
                                      int num_pages, const void* row_slot, const void* row_pos, int rows, int Hq, int Hkv,
                                      int D, float sm_scale, int kv_fp8, int split_tokens, int max_splits,
                                      int max_visible, const void* gate, int ld_gate, int gate_head_stride,
                                      int gate_offset, void* out, void* status, cudaStream_t stream) {
    using namespace ps;
    g_noalloc_err[0] = 0;
    if (rows <= 0 || Hq <= 0 || max_splits <= 0 || D <= 0) return (int)cudaErrorInvalidValue;
    const size_t acc_floats = (size_t)rows * Hq * max_splits * D;
    const size_t ml_floats = (size_t)rows * Hq * max_splits * 2;
    const size_t need = (acc_floats + ml_floats) * sizeof(float);
    if (need > (size_t)kNoAllocScratchBytes) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err),
                 "ps_paged_attention_noalloc: rows*Hq*max_splits*(D+2)*4 = %zu bytes exceeds the built-in scratch of %d bytes",
                 need, (int)kNoAllocScratchBytes);
        return PS_NOALLOC_TOO_LARGE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err), "ps_paged_attention_noalloc: cannot identify the current device");
        return PS_NOALLOC_SETUP_FAILED;
    }
    if (g_noalloc_ptr[dev] == nullptr) {
        // One-time set-up for this device: the array's name is only a host-side stand-in, the kernels
        // need its device address.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            snprintf(g_noalloc_err, sizeof(g_noalloc_err), "ps_paged_attention_noalloc: cudaGetSymbolAddress failed: %s",
                     cudaGetErrorString(e));
            return PS_NOALLOC_SETUP_FAILED;
        }
        g_noalloc_ptr[dev] = p;
    }
    float* part_acc = reinterpret_cast<float*>(g_noalloc_ptr[dev]);
    float* part_ml = part_acc + acc_floats;
    return ps_paged_attention(q, k_pool, v_pool, k_scale, v_scale, block_table, max_blocks, page_tokens, num_pages,
                              row_slot, row_pos, rows, Hq, Hkv, D, sm_scale, kv_fp8, split_tokens, max_splits, max_visible,
                              part_acc, part_ml, gate, ld_gate, gate_head_stride, gate_offset, out, status, stream);
}
