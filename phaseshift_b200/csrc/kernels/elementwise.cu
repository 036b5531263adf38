// Row-wise glue kernels used by the large-M (prefill) path and the model edges: embedding gather,
// RMSNorm(1+w), residual add, interleaved SwiGLU, row gather.  The decode path does not launch
// any of these except the embedding: they are folded into the small-M linear prologue/epilogue.
// Reference counterparts: src/phaseshift/models/qwen35/kernels/optimized/{embedding.hip:54,
// rmsnorm.hip:39, elementwise.hip:23-404, output_gather.hip:17}.
#include "ps_common.cuh"

namespace ps {

// out[r, :] = table[ids[r], :]; an id outside [0, vocab) writes zeros and flags the status word.
// `ssq` (optional): ssq[r * ssq_ld] receives the row's sum of squares, which lets the first projection's fused
// RMSNorm skip its own sweep over the row (see gemm_bs.cu).
__global__ void embedding_kernel(const int* ids, const __nv_bfloat16* table, int vocab, int H,
                                 __nv_bfloat16* out, int ldo, uint32_t* status, float* ssq, int ssq_ld) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int id = ids[r];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) set_status(status, PS_DEV_BAD_INDEX);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * ldo);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
        const uint4 v = ok ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
        dst[i] = v;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 a = bf16x2_bits_to_f32x2(w[e]); ss += a.x * a.x + a.y * a.y; }
    }
    if (ssq != nullptr) {
        ss = block_sum(ss, red);
        if (threadIdx.x == 0) ssq[(size_t)r * ssq_ld] = ss;
    }
}

// MXFP8 table (E4M3 codes + UE8M0 scale per 32): dequantising gather.
__global__ void embedding_mxfp8_kernel(const int* ids, const uint8_t* codes, const uint8_t* scales, int vocab,
                                       int H, __nv_bfloat16* out, int ldo, uint32_t* status, float* ssq, int ssq_ld) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int id = ids[r];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) set_status(status, PS_DEV_BAD_INDEX);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = 0.f;
        if (ok) v = e4m3_to_f32(codes[(size_t)id * H + i]) * __uint_as_float((uint32_t)scales[(size_t)id * (H / 32) + i / 32] << 23);
        const __nv_bfloat16 o = f32_to_bf16(v);
        out[(size_t)r * ldo + i] = o;
        const float of = bf16_to_f32(o);
        ss += of * of;
    }
    if (ssq != nullptr) {
        ss = block_sum(ss, red);
        if (threadIdx.x == 0) ssq[(size_t)r * ssq_ld] = ss;
    }
}

// y = bf16( x * rsqrt(mean(x^2) + eps) * (1 + w) ), optionally x = a + b first (writes the sum too).
__global__ void rmsnorm_kernel(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* add, int ld_add,
                               __nv_bfloat16* sum_out, int ld_sum, const __nv_bfloat16* w, float eps, int H,
                               __nv_bfloat16* out, int ldo, int one_plus) {
    extern __shared__ float xs[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = bf16_to_f32(x[(size_t)r * ldx + i]);
        if (add != nullptr) {
            v = bf16_to_f32(f32_to_bf16(v + bf16_to_f32(add[(size_t)r * ld_add + i])));
            if (sum_out != nullptr) sum_out[(size_t)r * ld_sum + i] = f32_to_bf16(v);
        }
        xs[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float wv = bf16_to_f32(w[i]);
        out[(size_t)r * ldo + i] = f32_to_bf16(xs[i] * inv * (one_plus ? 1.f + wv : wv));
    }
}

__global__ void add_kernel(const __nv_bfloat16* a, int lda, const __nv_bfloat16* b, int ldb, __nv_bfloat16* out,
                           int ldo, int H) {
    const int r = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= H) return;
    const float2 av = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(a + (size_t)r * lda + i));
    const float2 bv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(b + (size_t)r * ldb + i));
    *reinterpret_cast<uint32_t*>(out + (size_t)r * ldo + i) = f32x2_to_bf16x2_bits(av.x + bv.x, av.y + bv.y);
}

// gu [rows, 2I] with (gate_j, up_j) interleaved at (2j, 2j+1)  ->  out[rows, I] = silu(gate) * up
__global__ void swiglu_interleaved_kernel(const __nv_bfloat16* gu, int ld, __nv_bfloat16* out, int ldo, int I) {
    const int r = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= I) return;
    const float2 v = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(gu + (size_t)r * ld + 2 * j));
    out[(size_t)r * ldo + j] = f32_to_bf16(silu_f(v.x) * v.y);
}

// out[i, :] = src[rows[i], :] (16-byte units)
__global__ void gather_rows_kernel(const uint8_t* src, size_t src_pitch, const int* rows, uint8_t* dst,
                                   size_t dst_pitch, int row_bytes, int n_src_rows, uint32_t* status) {
    const int i = blockIdx.x;
    const int r = rows[i];
    if (r < 0 || r >= n_src_rows) { if (threadIdx.x == 0) set_status(status, PS_DEV_BAD_INDEX); return; }
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)r * src_pitch);
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)i * dst_pitch);
    for (int k = threadIdx.x; k < row_bytes / 16; k += blockDim.x) d[k] = s[k];
}

}  // namespace ps

PS_API int ps_embedding(const void* ids, const void* table, int rows, int vocab, int H, void* out, int ldo,
                        void* status, void* ssq, int ssq_ld, cudaStream_t stream) {
    if (rows <= 0 || (H % 8)) return (int)cudaErrorInvalidValue;
    ps::embedding_kernel<<<rows, 256, 0, stream>>>((const int*)ids, (const __nv_bfloat16*)table, vocab, H,
                                                   (__nv_bfloat16*)out, ldo, (uint32_t*)status, (float*)ssq, ssq_ld);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_embedding_mxfp8(const void* ids, const void* codes, const void* scales, int rows, int vocab, int H,
                              void* out, int ldo, void* status, void* ssq, int ssq_ld, cudaStream_t stream) {
    if (rows <= 0 || (H % 32)) return (int)cudaErrorInvalidValue;
    ps::embedding_mxfp8_kernel<<<rows, 256, 0, stream>>>((const int*)ids, (const uint8_t*)codes,
                                                         (const uint8_t*)scales, vocab, H, (__nv_bfloat16*)out, ldo,
                                                         (uint32_t*)status, (float*)ssq, ssq_ld);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_rmsnorm(const void* x, int ldx, const void* add, int ld_add, void* sum_out, int ld_sum, const void* w,
                      float eps, int rows, int H, void* out, int ldo, int one_plus, cudaStream_t stream) {
    if (rows <= 0 || H <= 0 || H > 32768) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(ps::rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        attr_set = true;
    }
    ps::rmsnorm_kernel<<<rows, 256, (size_t)H * 4, stream>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)add, ld_add, (__nv_bfloat16*)sum_out, ld_sum,
        (const __nv_bfloat16*)w, eps, H, (__nv_bfloat16*)out, ldo, one_plus);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_add(const void* a, int lda, const void* b, int ldb, void* out, int ldo, int rows, int H,
                  cudaStream_t stream) {
    if (rows <= 0 || (H & 1)) return (int)cudaErrorInvalidValue;
    dim3 grid((H / 2 + 255) / 256, rows);
    ps::add_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)b, ldb,
                                             (__nv_bfloat16*)out, ldo, H);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_swiglu_interleaved(const void* gu, int ld, void* out, int ldo, int rows, int I, cudaStream_t stream) {
    if (rows <= 0 || I <= 0) return (int)cudaErrorInvalidValue;
    dim3 grid((I + 255) / 256, rows);
    ps::swiglu_interleaved_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, ld, (__nv_bfloat16*)out, ldo, I);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_gather_rows(const void* src, long long src_pitch, const void* rows, int n, void* dst,
                          long long dst_pitch, int row_bytes, int n_src_rows, void* status, cudaStream_t stream) {
    if (n <= 0 || (row_bytes % 16)) return (int)cudaErrorInvalidValue;
    ps::gather_rows_kernel<<<n, 128, 0, stream>>>((const uint8_t*)src, (size_t)src_pitch, (const int*)rows,
                                                  (uint8_t*)dst, (size_t)dst_pitch, row_bytes, n_src_rows,
                                                  (uint32_t*)status);
    return PS_LAUNCH_CHECK();
}

// ---- library-wide budget of bounded device-side waits (declared in ps_common.cuh)
long long g_ps_wait_budget_cycles = 2000000000ll;

// Set the budget (GPU clock cycles) that launchers hand to kernels with bounded waits.  Values below 1000
// are clamped.  Returns the previous value.  Tests use a small budget to make a wait run out on purpose;
// deployments with slow peers may raise it.
PS_API long long ps_set_wait_budget(long long cycles) {
    const long long prev = g_ps_wait_budget_cycles;
    g_ps_wait_budget_cycles = cycles < 1000 ? 1000 : cycles;
    return prev;
}

// 1 when this library was compiled with -DPS_CHECKED (descriptor assertions on, see ps_common.cuh).
PS_API int ps_checked_build() {
#ifdef PS_CHECKED
    return 1;
#else
    return 0;
#endif
}
