// Offline-tooling kernels: NVFP4 / MXFP8 row quantisers (bit-equal to the CPU reference quantisers in
// csrc/runtime/io_quant.cpp: same scale search, same error metric in double, same tie rules), KL
// divergence / top-1 agreement / negative log-likelihood reductions over logits rows, and the
// importance-matrix accumulation.  Counterparts of the reference's offline kernels
// (src/phaseshift/quantization/offline/gpu_quantizer.hip:8-301, offline/gpu_kld.hip:34-115,
// imatrix/gpu_collector.hip:24).
#include "ps_common.cuh"

namespace ps {

__device__ __forceinline__ float q_e4m3_decode(uint32_t b) {
    const int s = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0) v = ldexpf((float)m, -9);
    else if (e == 15 && m == 7) v = __int_as_float(0x7fc00000);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return s ? -v : v;
}
__device__ __forceinline__ uint32_t q_e4m3_encode(float x) {     // nearest even, saturating to +-448
    if (x != x) return 0x7F;
    const uint32_t sign = signbit(x) ? 0x80u : 0u;
    const float a = fabsf(x);
    if (a >= 448.0f) return sign | 0x7E;
    if (a < ldexpf(1.0f, -10)) return sign;
    int e;
    frexpf(a, &e);
    int ex = e - 1;
    if (ex < -6) ex = -6;
    const float step = ldexpf(1.0f, ex - 3);
    const float q = a / step;
    float r = nearbyintf(q);
    if (r >= 16.0f) { r = 8.0f; ++ex; }
    if (ex > 8 || (ex == 8 && r > 14.0f)) return sign | 0x7E;
    uint32_t code;
    if (r < 8.0f) code = (uint32_t)r;
    else code = (uint32_t)(((ex + 7) << 3) | ((int)r - 8));
    return sign | code;
}
__device__ __forceinline__ float q_e2m1_decode(uint32_t nib) {
    const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float v = lut[nib & 7];
    return (nib & 8) ? -v : v;
}
__device__ __forceinline__ uint32_t q_e2m1_encode(float x) {
    const float bounds[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    const float a = fabsf(x);
    int idx = 0;
    while (idx < 7 && a > bounds[idx]) ++idx;
    if (idx < 7 && a == bounds[idx] && (idx & 1)) ++idx;
    if (idx == 0) return 0;
    return (uint32_t)(idx | (x < 0 ? 8 : 0));
}

// One thread per 16-weight block.
__global__ void quantize_nvfp4_kernel(const float* __restrict__ w, long long ldw, int N, int K, int k_padded, float tensor_scale,
                                      int search, const float* __restrict__ importance, uint8_t* __restrict__ codes,
                                      uint8_t* __restrict__ scales) {
    const int bpr = k_padded / 16;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (long long)N * bpr) return;
    const int row = (int)(id / bpr), b0 = (int)(id % bpr) * 16;
    float blk[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { blk[i] = (b0 + i < K) ? w[(long long)row * ldw + b0 + i] : 0.f; amax = fmaxf(amax, fabsf(blk[i])); }
    const int base = (int)q_e4m3_encode(amax / 6.0f / tensor_scale);
    double best_err = 0; int best_sb = 0; uint32_t best_lo = 0, best_hi = 0;
    bool have = false;
    for (int step = -search; step <= search; ++step) {
        const int sb = min(0x7E, max(0, base + step));
        const float s = q_e4m3_decode((uint32_t)sb) * tensor_scale;
        const float ss = s > 0 ? s : 1.0f;
        double err = 0; uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float r = blk[i] / ss;
            const uint32_t q = q_e2m1_encode(r);
            const float d = q_e2m1_decode(q) * s - blk[i];
            const float wgt = (importance != nullptr && b0 + i < K) ? importance[b0 + i] : 1.0f;
            err += (double)(d * d * wgt);
            if (i < 8) lo |= q << (4 * i); else hi |= q << (4 * (i - 8));
        }
        if (!have || err < best_err) { have = true; best_err = err; best_sb = sb; best_lo = lo; best_hi = hi; }
    }
    scales[(long long)row * bpr + b0 / 16] = (uint8_t)best_sb;
    uint32_t* cp = reinterpret_cast<uint32_t*>(codes + (long long)row * (k_padded / 2) + b0 / 2);
    cp[0] = best_lo; cp[1] = best_hi;
}

// One thread per 32-weight block.
__global__ void quantize_mxfp8_kernel(const float* __restrict__ w, long long ldw, int N, int K, int k_padded, int search,
                                      const float* __restrict__ importance, uint8_t* __restrict__ codes,
                                      uint8_t* __restrict__ scales) {
    const int bpr = k_padded / 32;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (long long)N * bpr) return;
    const int row = (int)(id / bpr), b0 = (int)(id % bpr) * 32;
    float blk[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { blk[i] = (b0 + i < K) ? w[(long long)row * ldw + b0 + i] : 0.f; amax = fmaxf(amax, fabsf(blk[i])); }
    int fe;
    const float fm = frexpf((amax > 0 ? amax : 1.0f) / 448.0f, &fe);
    const int e0 = fm == 0.5f ? fe - 1 : fe;
    double best_err = 0; int best_e = 0;
    bool have = false;
    for (int step = -search; step <= search; ++step) {
        const int e = min(127, max(-126, e0 + step));
        const float s = ldexpf(1.0f, e);
        double err = 0;
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
            const uint32_t c = q_e4m3_encode(blk[i] / s);
            const float d = q_e4m3_decode(c) * s - blk[i];
            const float wgt = (importance != nullptr && b0 + i < K) ? importance[b0 + i] : 1.0f;
            err += (double)(d * d * wgt);
        }
        if (!have || err < best_err) { have = true; best_err = err; best_e = e; }
    }
    const float s = ldexpf(1.0f, best_e);
    uint8_t* cp = codes + (long long)row * k_padded + b0;
#pragma unroll 8
    for (int i = 0; i < 32; ++i) cp[i] = (uint8_t)q_e4m3_encode(blk[i] / s);
    scales[(long long)row * bpr + b0 / 32] = (uint8_t)(best_e + 127);
}

// One CTA per row: KL(softmax(base) || softmax(cand)) in nats, top-1 agreement, and base-top-1 probability
// under the candidate.
__global__ void __launch_bounds__(512) kld_rows_kernel(const float* __restrict__ base, const float* __restrict__ cand, int vocab,
                                                        long long ld, float* __restrict__ out_kld, int* __restrict__ out_agree) {
    __shared__ float red[96];
    __shared__ int s_arg[2][16];
    __shared__ float s_val[2][16];
    const float* b = base + (long long)blockIdx.x * ld;
    const float* c = cand + (long long)blockIdx.x * ld;
    float mb = -3.0e38f, mc = -3.0e38f; int ab = 0, ac = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float vb = b[i], vc = c[i];
        if (vb > mb) { mb = vb; ab = i; }
        if (vc > mc) { mc = vc; ac = i; }
    }
    // block arg-max (ties -> lower index)
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, mb, o); const int oib = __shfl_xor_sync(0xffffffffu, ab, o);
        if (ob > mb || (ob == mb && oib < ab)) { mb = ob; ab = oib; }
        const float oc = __shfl_xor_sync(0xffffffffu, mc, o); const int oic = __shfl_xor_sync(0xffffffffu, ac, o);
        if (oc > mc || (oc == mc && oic < ac)) { mc = oc; ac = oic; }
    }
    const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { s_val[0][wp] = mb; s_arg[0][wp] = ab; s_val[1][wp] = mc; s_arg[1][wp] = ac; }
    __syncthreads();
    mb = s_val[0][0]; ab = s_arg[0][0]; mc = s_val[1][0]; ac = s_arg[1][0];
    for (int w2 = 1; w2 < nw; ++w2) {
        if (s_val[0][w2] > mb || (s_val[0][w2] == mb && s_arg[0][w2] < ab)) { mb = s_val[0][w2]; ab = s_arg[0][w2]; }
        if (s_val[1][w2] > mc || (s_val[1][w2] == mc && s_arg[1][w2] < ac)) { mc = s_val[1][w2]; ac = s_arg[1][w2]; }
    }
    float zb = 0.f, zc = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) { zb += __expf(b[i] - mb); zc += __expf(c[i] - mc); }
    float z2[2] = {zb, zc};
    block_sum_n<2>(z2, red);
    const float lzb = __logf(z2[0]) + mb, lzc = __logf(z2[1]) + mc;
    float kl = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float lpb = b[i] - lzb, lpc = c[i] - lzc;
        kl += __expf(lpb) * (lpb - lpc);
    }
    kl = block_sum(kl, red);
    if (threadIdx.x == 0) { out_kld[blockIdx.x] = fmaxf(kl, 0.f); out_agree[blockIdx.x] = ab == ac ? 1 : 0; }
}

// One CTA per row: -log softmax(logits)[target].
__global__ void __launch_bounds__(512) nll_rows_kernel(const float* __restrict__ logits, const int* __restrict__ target, int vocab,
                                                        long long ld, float* __restrict__ out) {
    __shared__ float red[64];
    const float* l = logits + (long long)blockIdx.x * ld;
    float m = -3.0e38f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, l[i]);
    m = block_max(m, red);
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += __expf(l[i] - m);
    z = block_sum(z, red + 32);
    if (threadIdx.x == 0) {
        const int t = target[blockIdx.x];
        out[blockIdx.x] = (t >= 0 && t < vocab) ? (__logf(z) + m - l[t]) : 0.f;
    }
}

// acc[k] += sum over rows of x[row, k]^2 (activation second moments at a projection input).
__global__ void imatrix_accumulate_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int rows, int K, float* __restrict__ acc) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= K) return;
    float s = 0.f;
    for (int r = 0; r < rows; ++r) { const float v = bf16_to_f32(x[(long long)r * ldx + k]); s = fmaf(v, v, s); }
    acc[k] += s;
}

}  // namespace ps

PS_API int ps_quantize_rows(int fmt_nvfp4, const void* w, long long ldw, int N, int K, int k_padded, float tensor_scale,
                            int search, const void* importance, void* codes, void* scales, cudaStream_t stream) {
    using namespace ps;
    if (N <= 0 || K <= 0 || k_padded < K || search < 0) return (int)cudaErrorInvalidValue;
    if (fmt_nvfp4) {
        if (k_padded % 16 || !(tensor_scale > 0.f)) return (int)cudaErrorInvalidValue;
        const long long n = (long long)N * (k_padded / 16);
        quantize_nvfp4_kernel<<<(unsigned)((n + 127) / 128), 128, 0, stream>>>((const float*)w, ldw, N, K, k_padded, tensor_scale, search,
                                                                               (const float*)importance, (uint8_t*)codes, (uint8_t*)scales);
    } else {
        if (k_padded % 32) return (int)cudaErrorInvalidValue;
        const long long n = (long long)N * (k_padded / 32);
        quantize_mxfp8_kernel<<<(unsigned)((n + 127) / 128), 128, 0, stream>>>((const float*)w, ldw, N, K, k_padded, search,
                                                                               (const float*)importance, (uint8_t*)codes, (uint8_t*)scales);
    }
    return PS_LAUNCH_CHECK();
}

PS_API int ps_kld_rows(const void* base, const void* cand, int rows, int vocab, long long ld, void* out_kld, void* out_agree,
                       cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return (int)cudaErrorInvalidValue;
    ps::kld_rows_kernel<<<rows, 512, 0, stream>>>((const float*)base, (const float*)cand, vocab, ld, (float*)out_kld, (int*)out_agree);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_nll_rows(const void* logits, const void* target, int rows, int vocab, long long ld, void* out, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return (int)cudaErrorInvalidValue;
    ps::nll_rows_kernel<<<rows, 512, 0, stream>>>((const float*)logits, (const int*)target, vocab, ld, (float*)out);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_imatrix_accumulate(const void* x, long long ldx, int rows, int K, void* acc, cudaStream_t stream) {
    if (rows <= 0 || K <= 0) return (int)cudaErrorInvalidValue;
    ps::imatrix_accumulate_kernel<<<(K + 255) / 256, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, rows, K, (float*)acc);
    return PS_LAUNCH_CHECK();
}
