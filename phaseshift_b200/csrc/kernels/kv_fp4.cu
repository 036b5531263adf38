// Attention over NVFP4 key/value pages (row format in kv_fp4.cuh).
//
//   * ps_paged_attention_fp4: the split-KV partial pass for decode / verify rows.  Same work split, shared-memory
//     tiles, summation order and partial layout as the bf16 / FP8 kernel of paged_attention.cu (one CTA = (split,
//     KV head, row), 32-token tiles, all query heads of the group served from one tile), so its partials go through the
//     same merge pass (ps_paged_attention_merge).  A tile of a 256-wide head is 32 x 144 bytes: every thread fetches one
//     16-byte piece of codes (32 values) and the two block scales that belong to it, and widens them to bf16 on the way
//     into shared memory (exact); the per-token fp32 scale multiplies the score and the probability, as for FP8 pages.
//     It is a kernel of its own rather than a third branch of that one, so that adding the format left the code generated
//     for the bf16 / FP8 kernel (whose timings are on record) exactly as it was.
//   * ps_kv_fp4_dequant: widens the pages that a prefill step reads into a bf16 scratch pool with a block table and
//     sequence descriptors of its own, on which the tiled tensor-core prefill kernels run unchanged (the same scheme the
//     FP8 pools use).  4.6 bits are read and 16 written per cached value, once per layer and step.
//
// Reference counterparts: the PSQ4 KV read paths of src/phaseshift/models/qwen35/kernels/optimized/attention/
// paged_decode.hip:264-300 and paged_prefill.hip (KV dtype dispatch).
#include "kv_fp4.cuh"

namespace ps {

constexpr int kF4Tile = 32;        // tokens per shared-memory tile
constexpr int kF4Threads = 256;
constexpr int kF4MaxG = 8;
constexpr int kF4MaxD = 256;
constexpr int kF4MaxSplits = 1024;

struct Fp4AttnArgs {
    const __nv_bfloat16* q;      // [rows, Hq, D]
    const uint8_t* k_pool; const uint8_t* v_pool; const float* k_scale; const float* v_scale;
    const int* block_table; int max_blocks; int page_tokens; int num_pages;
    const int* row_slot; const int* row_pos;
    int rows, Hq, Hkv, D; float sm_scale;
    int split_tokens, max_splits;
    float* part_acc;   // [rows, Hq, max_splits, D]
    float* part_ml;    // [rows, Hq, max_splits, 2]  (running max, running sum)
    uint32_t* status;
};

struct Fp4TileRegs { uint4 k, v; uint32_t ksf, vsf; float ks, vs; };

// Thread t < 32 * D/32 owns piece (token t / (D/32), 32-value group t % (D/32)) of the tile.
__device__ __forceinline__ void fp4_tile_fetch(const Fp4AttnArgs& a, Fp4TileRegs& r, int slot, int kvh, int tok0, int visible,
                                               bool& bad) {
    const int ppr = a.D / 32, row_bytes = kv_fp4_row_bytes(a.D);
    r.k = make_uint4(0, 0, 0, 0); r.v = make_uint4(0, 0, 0, 0); r.ksf = 0; r.vsf = 0; r.ks = 1.f; r.vs = 1.f;
    const int p = threadIdx.x;
    if (p < kF4Tile * ppr) {
        const int t = p / ppr, c = p % ppr;
        const int tok = tok0 + t;
        if (tok < visible) {
            const int page = a.block_table[(size_t)slot * a.max_blocks + tok / a.page_tokens];
            if (page < 0 || page >= a.num_pages) { bad = true; }
            else {
                const size_t off = (((size_t)page * a.Hkv + kvh) * a.page_tokens + tok % a.page_tokens) * row_bytes;
                r.k = __ldg(reinterpret_cast<const uint4*>(a.k_pool + off + c * 16));
                r.v = __ldg(reinterpret_cast<const uint4*>(a.v_pool + off + c * 16));
                r.ksf = __ldg(reinterpret_cast<const unsigned short*>(a.k_pool + off + a.D / 2 + 2 * c));
                r.vsf = __ldg(reinterpret_cast<const unsigned short*>(a.v_pool + off + a.D / 2 + 2 * c));
            }
        }
    }
    if (threadIdx.x < kF4Tile) {
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

__device__ __forceinline__ void fp4_tile_store(const Fp4AttnArgs& a, const Fp4TileRegs& r, __nv_bfloat16* ks, __nv_bfloat16* vs,
                                               float* kscale, float* vscale) {
    const int ppr = a.D / 32, kpitch = a.D + 8;
    const int p = threadIdx.x;
    if (p < kF4Tile * ppr) {
        const int t = p / ppr, c = p % ppr;
        uint4 o[4];
        kv_fp4_piece_to_bf16(r.k, r.ksf, o);
        uint4* kd = reinterpret_cast<uint4*>(ks + t * kpitch + c * 32);
        kd[0] = o[0]; kd[1] = o[1]; kd[2] = o[2]; kd[3] = o[3];
        kv_fp4_piece_to_bf16(r.v, r.vsf, o);
        uint4* vd = reinterpret_cast<uint4*>(vs + t * a.D + c * 32);
        vd[0] = o[0]; vd[1] = o[1]; vd[2] = o[2]; vd[3] = o[3];
    }
    if (threadIdx.x < kF4Tile) { kscale[threadIdx.x] = r.ks; vscale[threadIdx.x] = r.vs; }
}

__global__ void __launch_bounds__(kF4Threads) paged_attn_split_fp4_kernel(const Fp4AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int D = a.D, G = a.Hq / a.Hkv, kpitch = D + 8;
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem);            // [32][D+8]
    __nv_bfloat16* vs = ks + kF4Tile * kpitch;                             // [32][D]
    float* qs = reinterpret_cast<float*>(vs + kF4Tile * D);                // [G][D]
    float* ps_ = qs + kF4MaxG * D;                                         // [G][32]
    float* alpha = ps_ + kF4MaxG * kF4Tile;                                // [G]
    float* kscale = alpha + kF4MaxG;                                       // [32]
    float* vscale = kscale + kF4Tile;                                      // [32]

    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();
    const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int visible = a.row_pos[row] + 1;
    const int tok_begin = split * a.split_tokens;
    if (tok_begin >= visible) return;
    const int tok_end = min(visible, tok_begin + a.split_tokens);
    const int slot = a.row_slot[row];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

    for (int i = t; i < G * D; i += kF4Threads) {
        const int g = i / D, d = i % D;
        qs[i] = bf16_to_f32(a.q[((size_t)row * a.Hq + kvh * G + g) * D + d]) * a.sm_scale;
    }
    float acc[kF4MaxG];
#pragma unroll
    for (int g = 0; g < kF4MaxG; ++g) acc[g] = 0.f;
    float m_run = -3.0e38f, l_run = 0.f;   // owned by warp g (all lanes hold the same value)

    bool bad = false;
    Fp4TileRegs regs;
    fp4_tile_fetch(a, regs, slot, kvh, tok_begin, tok_end, bad);
    for (int tok0 = tok_begin; tok0 < tok_end; tok0 += kF4Tile) {
        __syncthreads();                       // previous tile fully consumed
        fp4_tile_store(a, regs, ks, vs, kscale, vscale);
        __syncthreads();
        if (tok0 + kF4Tile < tok_end) fp4_tile_fetch(a, regs, slot, kvh, tok0 + kF4Tile, tok_end, bad);

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
            ps_[warp * kF4Tile + lane] = p * vscale[lane];
            if (lane == 0) alpha[warp] = al;
        }
        __syncthreads();
        // PV: thread = output dim, all heads; tokens outermost, four at a time
        if (t < D) {
#pragma unroll
            for (int g = 0; g < kF4MaxG; ++g)
                if (g < G) acc[g] *= alpha[g];
#pragma unroll 2
            for (int j0 = 0; j0 < kF4Tile; j0 += 4) {
                float vv[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) vv[jj] = bf16_to_f32(vs[(j0 + jj) * D + t]);
#pragma unroll
                for (int g = 0; g < kF4MaxG; ++g) {
                    if (g < G) {
                        const float4 pq = *reinterpret_cast<const float4*>(ps_ + g * kF4Tile + j0);
                        float s = acc[g];
                        s = fmaf(pq.x, vv[0], s); s = fmaf(pq.y, vv[1], s); s = fmaf(pq.z, vv[2], s); s = fmaf(pq.w, vv[3], s);
                        acc[g] = s;
                    }
                }
            }
        }
    }
    if (bad && t == 0) set_status(a.status, PS_DEV_BAD_INDEX);
    if (t < D) {
#pragma unroll
        for (int g = 0; g < kF4MaxG; ++g)
            if (g < G) a.part_acc[(((size_t)row * a.Hq + kvh * G + g) * a.max_splits + split) * D + t] = acc[g];
    }
    if (warp < G && lane == 0) {
        float* ml = a.part_ml + (((size_t)row * a.Hq + kvh * G + warp) * a.max_splits + split) * 2;
        ml[0] = m_run; ml[1] = l_run;
    }
}

struct Fp4DeqArgs {
    const uint8_t* k_pool; const uint8_t* v_pool; const float* k_scale; const float* v_scale;
    const int* block_table; int max_blocks; int num_pages; int page_tokens; int Hkv; int D;
    const int* seqs; int n_seqs; int min_rows;
    __nv_bfloat16* k_out; __nv_bfloat16* v_out;
    int* bt_out;                 // [n_seqs][max_blocks]
    int* seqs_out;               // [n_seqs][4]
    uint32_t* status;
};

// grid = (scratch pages, Hkv), block = 256.  Scratch page p belongs to the p-th page of the step's long sequences taken in
// order (sequences with at most `min_rows` rows are served by the per-row kernel and skipped here); the scratch block
// table maps (sequence index, block) to it and the scratch descriptors carry the sequence index as the slot.
__global__ void __launch_bounds__(256) kv_fp4_dequant_kernel(const Fp4DeqArgs a) {
    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();
    const int p = blockIdx.x, kvh = blockIdx.y, pt = a.page_tokens, D = a.D;
    int base = 0, s = 0, blk = -1, kv_end = 0, slot = -1;
    for (; s < a.n_seqs; ++s) {
        const int* sd = a.seqs + 4 * s;
        const int n_rows = sd[1];
        if (sd[2] < 0 || n_rows <= a.min_rows) continue;
        const int end = sd[3] + n_rows, np = (end + pt - 1) / pt;
        if (p < base + np) { blk = p - base; kv_end = end; slot = sd[2]; break; }
        base += np;
    }
    if (p == 0 && kvh == 0) {
        for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x) {
            const int* sd = a.seqs + 4 * i;
            a.seqs_out[4 * i + 0] = sd[0]; a.seqs_out[4 * i + 1] = sd[1]; a.seqs_out[4 * i + 2] = sd[2] < 0 ? -1 : i;
            a.seqs_out[4 * i + 3] = sd[3];
        }
    }
    if (blk < 0) return;
    if (kvh == 0 && threadIdx.x == 0) a.bt_out[(size_t)s * a.max_blocks + blk] = p;
    const int page = (blk < a.max_blocks) ? a.block_table[(size_t)slot * a.max_blocks + blk] : -1;
    const bool ok = page >= 0 && page < a.num_pages;
    if (!ok && threadIdx.x == 0) set_status(a.status, PS_DEV_BAD_INDEX);
    const int ppr = D / 32, row_bytes = kv_fp4_row_bytes(D);
    const size_t src = ((size_t)(ok ? page : 0) * a.Hkv + kvh) * pt;          // token rows of the source page
    const size_t dst = ((size_t)p * a.Hkv + kvh) * pt;
    for (int i = threadIdx.x; i < pt * ppr; i += blockDim.x) {
        const int tok = i / ppr, c = i % ppr;
        const bool live = ok && blk * pt + tok < kv_end;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const uint8_t* pool = which ? a.v_pool : a.k_pool;
            const float* sp = which ? a.v_scale : a.k_scale;
            __nv_bfloat16* out = which ? a.v_out : a.k_out;
            uint4 o[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            if (live) {
                const uint8_t* rowp = pool + (src + tok) * row_bytes;
                const uint4 cw = __ldg(reinterpret_cast<const uint4*>(rowp + c * 16));
                const uint32_t sf2 = __ldg(reinterpret_cast<const unsigned short*>(rowp + D / 2 + 2 * c));
                const float ts = sp[src + tok];
                const float s0 = e4m3_to_f32((uint8_t)(sf2 & 0xffu)) * ts, s1 = e4m3_to_f32((uint8_t)(sf2 >> 8)) * ts;
                const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
                uint32_t ob[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((w[j >> 2] >> ((j & 3) * 8)) & 0xffu), __NV_E2M1);
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
                    const float sc = j < 8 ? s0 : s1;
                    ob[j] = f32x2_to_bf16x2_bits(f.x * sc, f.y * sc);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) o[q] = make_uint4(ob[4 * q], ob[4 * q + 1], ob[4 * q + 2], ob[4 * q + 3]);
            }
            uint4* d = reinterpret_cast<uint4*>(out + (dst + tok) * D + c * 32);
            d[0] = o[0]; d[1] = o[1]; d[2] = o[2]; d[3] = o[3];
        }
    }
}

}  // namespace ps

// Split-KV partial pass over NVFP4 pages; finish with ps_paged_attention_merge(part_acc, part_ml, row_pos, ...).
PS_API int ps_paged_attention_fp4(const void* q, const void* k_pool, const void* v_pool, const void* k_scale,
                                  const void* v_scale, const void* block_table, int max_blocks, int page_tokens,
                                  int num_pages, const void* row_slot, const void* row_pos, int rows, int Hq, int Hkv,
                                  int D, float sm_scale, int split_tokens, int max_splits, int max_visible,
                                  void* part_acc, void* part_ml, void* status, cudaStream_t stream) {
    using namespace ps;
    const int G = Hkv > 0 ? Hq / Hkv : 0;
    if (G < 1 || G > kF4MaxG || (Hq % Hkv) || D > kF4MaxD || D < 32 || (D % 32) || (split_tokens % kF4Tile) || rows <= 0 ||
        k_scale == nullptr || v_scale == nullptr || ((uintptr_t)k_pool % 16) || ((uintptr_t)v_pool % 16))
        return (int)cudaErrorInvalidValue;
    Fp4AttnArgs a;
    a.q = (const __nv_bfloat16*)q; a.k_pool = (const uint8_t*)k_pool; a.v_pool = (const uint8_t*)v_pool;
    a.k_scale = (const float*)k_scale; a.v_scale = (const float*)v_scale; a.block_table = (const int*)block_table;
    a.max_blocks = max_blocks; a.page_tokens = page_tokens; a.num_pages = num_pages; a.row_slot = (const int*)row_slot;
    a.row_pos = (const int*)row_pos; a.rows = rows; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.sm_scale = sm_scale;
    a.split_tokens = split_tokens; a.max_splits = max_splits;
    a.part_acc = (float*)part_acc; a.part_ml = (float*)part_ml; a.status = (uint32_t*)status;
    int n_splits = (max_visible + split_tokens - 1) / split_tokens;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > max_splits || max_splits > kF4MaxSplits) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)kF4Tile * (D + 8) * 2 + (size_t)kF4Tile * D * 2 +
                        sizeof(float) * (kF4MaxG * D + kF4MaxG * kF4Tile + kF4MaxG + 2 * kF4Tile);
    return launch_pdl(paged_attn_split_fp4_kernel, dim3(n_splits, Hkv, rows), dim3(kF4Threads), smem, stream, a);
}

// Widen the NVFP4 pages of the step's sequences with more than `min_rows` rows into bf16 scratch pools of `out_pages` pages.
PS_API int ps_kv_fp4_dequant(const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale,
                             const void* block_table, int max_blocks, int num_pages, int page_tokens, int Hkv, int D,
                             const void* seqs, int n_seqs, int min_rows, void* k_out, void* v_out, int out_pages,
                             void* bt_out, void* seqs_out, void* status, cudaStream_t stream) {
    using namespace ps;
    if (out_pages <= 0 || Hkv <= 0 || D < 32 || (D % 32) || n_seqs <= 0 || k_scale == nullptr || v_scale == nullptr ||
        ((uintptr_t)k_pool % 16) || ((uintptr_t)v_pool % 16) || ((uintptr_t)k_out % 16) || ((uintptr_t)v_out % 16))
        return (int)cudaErrorInvalidValue;
    Fp4DeqArgs a;
    a.k_pool = (const uint8_t*)k_pool; a.v_pool = (const uint8_t*)v_pool; a.k_scale = (const float*)k_scale;
    a.v_scale = (const float*)v_scale; a.block_table = (const int*)block_table; a.max_blocks = max_blocks;
    a.num_pages = num_pages; a.page_tokens = page_tokens; a.Hkv = Hkv; a.D = D; a.seqs = (const int*)seqs; a.n_seqs = n_seqs;
    a.min_rows = min_rows; a.k_out = (__nv_bfloat16*)k_out; a.v_out = (__nv_bfloat16*)v_out; a.bt_out = (int*)bt_out;
    a.seqs_out = (int*)seqs_out; a.status = (uint32_t*)status;
    return launch_pdl(kv_fp4_dequant_kernel, dim3(out_pages, Hkv), dim3(256), 0, stream, a);
}
