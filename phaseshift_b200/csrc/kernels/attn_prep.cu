// Fused attention prepare: per-head RMSNorm(1+w) on q and k, partial NeoX RoPE, and the paged
// KV append (BF16, FP8-E4M3 with one f32 scale per token x kv-head, or NVFP4 rows as laid out in kv_fp4.cuh), in one launch.
//
// The reference runs these as separate dispatches (split, two per-group RMSNorms, RoPE pair
// kernel with an f64 inv_freq table, kv_append; src/phaseshift/models/qwen35/kernels/optimized/
// attention/rope.hip:130-251, kv_append.hip:98-148).  Here one CTA owns one (row, head): the
// normalised, rotated q is written to the dense q buffer, k/v go straight into their page.
//
// Layouts
//   qkv      [rows, ld_qkv] bf16: per q-head h: [2hD, 2hD+D) = q, [2hD+D, 2hD+2D) = gate;
//            then k heads at q_span + hk*D, then v heads at q_span + Hkv*D + hk*D.
//   q_out    [rows, Hq, D] bf16
//   k/v pool [num_pages, Hkv, page_tokens, D] (bf16 or e4m3) or [num_pages, Hkv, page_tokens, kv_fp4_row_bytes(D)] bytes
//            (NVFP4, kv_fp8 == 2), scales [num_pages, Hkv, page_tokens] f32
//   block_table [num_slots, max_blocks] int32; row_slot/row_pos give each row's sequence slot and position.
#include "kv_fp4.cuh"

namespace ps {

struct AttnPrepArgs {
    const __nv_bfloat16* qkv; int ld_qkv;
    int rows, Hq, Hkv, D, rotary_dim;
    const __nv_bfloat16* q_norm_w; const __nv_bfloat16* k_norm_w; float eps;
    const double* inv_freq;            // [rotary_dim/2]
    const int* row_slot; const int* row_pos;
    __nv_bfloat16* q_out;
    void* k_pool; void* v_pool; float* k_scale; float* v_scale;
    const int* block_table; int max_blocks; int page_tokens; int num_pages; int kv_fp8;
    uint32_t* status;
};

// grid = (Hq + 2*Hkv, rows), block = D/2 threads (each thread owns the NeoX pair (i, i + rot/2) for
// i < rot/2 and two plain elements otherwise).  D <= 512.
__global__ void attn_prep_kernel(const AttnPrepArgs a) {
    __shared__ float red[32];
    __shared__ float vals[512];
    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();
    const int row = blockIdx.y, hh = blockIdx.x, t = threadIdx.x, D = a.D;
    const int q_span = 2 * a.Hq * D;
    const __nv_bfloat16* src;
    int kind;  // 0 q, 1 k, 2 v
    int head;
    if (hh < a.Hq) { kind = 0; head = hh; src = a.qkv + (size_t)row * a.ld_qkv + 2 * head * D; }
    else if (hh < a.Hq + a.Hkv) { kind = 1; head = hh - a.Hq; src = a.qkv + (size_t)row * a.ld_qkv + q_span + head * D; }
    else { kind = 2; head = hh - a.Hq - a.Hkv; src = a.qkv + (size_t)row * a.ld_qkv + q_span + (a.Hkv + head) * D; }

    float x0 = bf16_to_f32(src[t]), x1 = bf16_to_f32(src[t + D / 2]);
    if (kind != 2) {
        const float ss = block_sum(x0 * x0 + x1 * x1, red);
        const float ir = rsqrtf(ss / (float)D + a.eps);
        const __nv_bfloat16* w = kind == 0 ? a.q_norm_w : a.k_norm_w;
        x0 = x0 * ir * (1.f + bf16_to_f32(w[t]));
        x1 = x1 * ir * (1.f + bf16_to_f32(w[t + D / 2]));
    }
    vals[t] = x0; vals[t + D / 2] = x1;
    __syncthreads();
    const int pos = a.row_pos[row];
    if (kind != 2) {
        const int half = a.rotary_dim / 2;
        if (t < half) {
            // NeoX half-rotate on the first rotary_dim dims: (x[i], x[i+half]) rotated by pos * inv_freq[i]
            double s, c;
            sincos((double)pos * a.inv_freq[t], &s, &c);
            const float lo = vals[t], hi = vals[t + half];
            // each (i, i+half) pair is read and rewritten by exactly one thread
            vals[t] = (float)((double)lo * c - (double)hi * s);
            vals[t + half] = (float)((double)hi * c + (double)lo * s);
        }
    }
    __syncthreads();
    if (kind == 0) {
        __nv_bfloat16* dst = a.q_out + ((size_t)row * a.Hq + head) * D;
        dst[t] = f32_to_bf16(vals[t]);
        dst[t + D / 2] = f32_to_bf16(vals[t + D / 2]);
        return;
    }
    const int slot = a.row_slot[row];
    if (slot < 0) return;   // padding row of a row bucket: nothing to append
    const int blk = pos / a.page_tokens, off = pos % a.page_tokens;
    if (blk >= a.max_blocks || pos < 0) { if (t == 0) set_status(a.status, PS_DEV_BAD_INDEX); return; }
    const int page = a.block_table[(size_t)slot * a.max_blocks + blk];
    if (page < 0 || page >= a.num_pages) { if (t == 0) set_status(a.status, PS_DEV_BAD_INDEX); return; }
    const size_t tok = ((size_t)page * a.Hkv + head) * a.page_tokens + off;
    void* pool = kind == 1 ? a.k_pool : a.v_pool;
    // K is stored after bf16 rounding of the rotated value, V as given.
    const float y0 = bf16_to_f32(f32_to_bf16(vals[t])), y1 = bf16_to_f32(f32_to_bf16(vals[t + D / 2]));
    if (!a.kv_fp8) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pool) + tok * D;
        dst[t] = f32_to_bf16(y0); dst[t + D / 2] = f32_to_bf16(y1);
    } else if (a.kv_fp8 == 2) {
        // NVFP4 row: token scale from the row maximum, then one thread per block of 16 values
        const float ts = kv_fp4_token_scale(block_max(fmaxf(fabsf(y0), fabsf(y1)), red));
        vals[t] = y0; vals[t + D / 2] = y1;          // each thread rewrites the two entries it alone has read
        __syncthreads();
        uint8_t* dst = reinterpret_cast<uint8_t*>(pool) + tok * kv_fp4_row_bytes(D);
        if (t < D / 16) {
            uint2 codes; uint8_t sf;
            kv_fp4_quant16(vals + 16 * t, ts, codes, sf);
            *reinterpret_cast<uint2*>(dst + 8 * t) = codes;
            dst[D / 2 + t] = sf;
        }
        if (t == 0) (kind == 1 ? a.k_scale : a.v_scale)[tok] = ts;
    } else {
        const float amax = block_max(fmaxf(fabsf(y0), fabsf(y1)), red);
        const float sc = amax > 0.f ? amax / 448.f : 1.f;
        const float inv = 1.f / sc;
        uint8_t* dst = reinterpret_cast<uint8_t*>(pool) + tok * D;
        dst[t] = f32_to_e4m3(y0 * inv); dst[t + D / 2] = f32_to_e4m3(y1 * inv);
        if (t == 0) (kind == 1 ? a.k_scale : a.v_scale)[tok] = sc;
    }
}

}  // namespace ps

PS_API int ps_attn_prep(const void* qkv, int ld_qkv, int rows, int Hq, int Hkv, int D, int rotary_dim,
                        const void* q_norm_w, const void* k_norm_w, float eps, const void* inv_freq,
                        const void* row_slot, const void* row_pos, void* q_out, void* k_pool, void* v_pool,
                        void* k_scale, void* v_scale, const void* block_table, int max_blocks, int page_tokens,
                        int num_pages, int kv_fp8, void* status, cudaStream_t stream) {
    using namespace ps;
    if (D > 512 || (D & 63) || rotary_dim > D || rows <= 0) return (int)cudaErrorInvalidValue;
    AttnPrepArgs a;
    a.qkv = (const __nv_bfloat16*)qkv; a.ld_qkv = ld_qkv; a.rows = rows; a.Hq = Hq; a.Hkv = Hkv; a.D = D;
    a.rotary_dim = rotary_dim; a.q_norm_w = (const __nv_bfloat16*)q_norm_w; a.k_norm_w = (const __nv_bfloat16*)k_norm_w;
    a.eps = eps; a.inv_freq = (const double*)inv_freq; a.row_slot = (const int*)row_slot; a.row_pos = (const int*)row_pos;
    a.q_out = (__nv_bfloat16*)q_out; a.k_pool = k_pool; a.v_pool = v_pool; a.k_scale = (float*)k_scale;
    a.v_scale = (float*)v_scale; a.block_table = (const int*)block_table; a.max_blocks = max_blocks;
    a.page_tokens = page_tokens; a.num_pages = num_pages; a.kv_fp8 = kv_fp8; a.status = (uint32_t*)status;
    dim3 grid(Hq + 2 * Hkv, rows);
    return launch_pdl(attn_prep_kernel, grid, dim3(D / 2), 0, stream, a);
}
