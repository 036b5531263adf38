// On-device sampling: greedy argmax, Gumbel-max with top-k / top-p membership tests, constraint
// bitmask.  Logits never leave the device (reference contract: docs/developer/sampling.md:225-239;
// reference kernels: src/phaseshift/models/qwen35/kernels/optimized/sampling.hip:102-290,
// stochastic_sampling.hip:13-56).  One CTA of 1024 threads per output row; the vocabulary is swept
// with coalesced loads, so the cost is one to three passes over a 600 KB logits row.
#include "ps_common.cuh"
#include "ps_sampling.h"

namespace ps {

constexpr int kSampThreads = 1024;

struct SampleArgs {
    const float* logits; int ld; int vocab; int rows;
    const SamplingRow* params;
    const uint32_t* mask; int mask_words;   // optional [rows, mask_words]; bit set = token allowed
    const uint8_t* mask_active;             // optional [rows]
    int* out;                               // [rows]; -1 on failure / empty constraint
    uint32_t* status;
};

__device__ __forceinline__ bool allowed(const uint32_t* m, uint32_t tok) {
    return m == nullptr || ((m[tok >> 5] >> (tok & 31u)) & 1u);
}

struct Best { float v; uint32_t i; };

__device__ __forceinline__ Best block_best(Best b, Best* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (ranks_before(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = b;
    __syncthreads();
    Best r = lane < (blockDim.x >> 5) ? sh[lane] : Best{-INFINITY, 0xffffffffu};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, r.v, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, r.i, o);
        if (ranks_before(ov, oi, r.v, r.i)) { r.v = ov; r.i = oi; }
    }
    return r;
}

__device__ __forceinline__ double block_sum_d(double v, double* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    double r = lane < (blockDim.x >> 5) ? sh[lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

__global__ void __launch_bounds__(kSampThreads) sample_kernel(const SampleArgs a) {
    __shared__ Best sh_best[32];
    __shared__ double sh_d[32];
    const int row = blockIdx.x;
    const SamplingRow p = a.params[row];
    if (p.mode == kSamplingNone) { if (threadIdx.x == 0) a.out[row] = -1; return; }
    const float* lg = a.logits + (size_t)row * a.ld;
    const uint32_t* m = (a.mask != nullptr && (a.mask_active == nullptr || a.mask_active[row]))
                            ? a.mask + (size_t)row * a.mask_words : nullptr;
    // pass 1: constrained argmax (also the softmax max); non-finite logits fail closed
    Best b{-INFINITY, 0xffffffffu};
    bool bad = false;
    if ((a.ld & 3) == 0 && (reinterpret_cast<uintptr_t>(a.logits) & 15) == 0) {
        // 16-byte loads, several in flight per thread: the sweep is latency-bound otherwise
        const uint32_t n4 = (uint32_t)a.vocab >> 2;
        const float4* lg4 = reinterpret_cast<const float4*>(lg);
#pragma unroll 4
        for (uint32_t j = threadIdx.x; j < n4; j += kSampThreads) {
            const float4 q = lg4[j];
            const float vv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t i = 4 * j + e;
                if (!(fabsf(vv[e]) <= 3.0e38f)) bad = true;
                if (allowed(m, i) && ranks_before(vv[e], i, b.v, b.i)) { b.v = vv[e]; b.i = i; }
            }
        }
        for (uint32_t i = 4 * n4 + threadIdx.x; i < (uint32_t)a.vocab; i += kSampThreads) {
            const float v = lg[i];
            if (!(fabsf(v) <= 3.0e38f)) bad = true;
            if (allowed(m, i) && ranks_before(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < (uint32_t)a.vocab; i += kSampThreads) {
            const float v = lg[i];
            if (!(fabsf(v) <= 3.0e38f)) bad = true;
            if (allowed(m, i) && ranks_before(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
    }
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    b = block_best(b, sh_best);
    if (any_bad || b.i == 0xffffffffu) {
        if (threadIdx.x == 0) {
            a.out[row] = -1;
            if (any_bad) set_status(a.status, PS_DEV_NONFINITE);
        }
        return;
    }
    if (p.mode == kSamplingGreedy || !(p.temperature > 0.f)) { if (threadIdx.x == 0) a.out[row] = (int)b.i; return; }

    const float inv_t = 1.f / p.temperature, mx = b.v;
    const bool need_mass = p.top_p < 1.f;
    double Z = 0.0;
    if (need_mass) {
        double z = 0.0;
        for (uint32_t i = threadIdx.x; i < (uint32_t)a.vocab; i += kSampThreads)
            if (allowed(m, i)) z += (double)__expf((lg[i] - mx) * inv_t);
        Z = block_sum_d(z, sh_d);
    }
    for (uint32_t attempt = 0; attempt < kMaxSamplingAttempts; ++attempt) {
        Best c{-INFINITY, 0xffffffffu};
        for (uint32_t i = threadIdx.x; i < (uint32_t)a.vocab; i += kSampThreads) {
            if (!allowed(m, i)) continue;
            const float u = sampling_uniform(p.seed, p.sample_index, attempt, i);
            const float s = (lg[i] - mx) * inv_t - logf(-logf(u));
            if (ranks_before(s, i, c.v, c.i)) { c.v = s; c.i = i; }
        }
        c = block_best(c, sh_best);
        bool ok = true;
        if (p.top_k > 0 || need_mass) {
            const float lc = lg[c.i];
            uint32_t cnt = 0; double mass = 0.0;
            for (uint32_t i = threadIdx.x; i < (uint32_t)a.vocab; i += kSampThreads) {
                if (!allowed(m, i)) continue;
                const float v = lg[i];
                if (ranks_before(v, i, lc, c.i)) { ++cnt; if (need_mass) mass += (double)__expf((v - mx) * inv_t); }
            }
            const double tot_cnt = block_sum_d((double)cnt, sh_d);
            if (p.top_k > 0 && tot_cnt >= (double)p.top_k) ok = false;
            if (need_mass) {
                const double tot_mass = block_sum_d(mass, sh_d);
                if (!(tot_mass < (double)p.top_p * Z)) ok = false;
            }
        }
        if (ok) { if (threadIdx.x == 0) a.out[row] = (int)c.i; return; }
    }
    if (threadIdx.x == 0) { a.out[row] = -1; set_status(a.status, PS_DEV_SAMPLING_FAILED); }
}

// Per-row argmax plus the runner-up margin (used by speculative heads to rank draft confidence).
__global__ void __launch_bounds__(kSampThreads) argmax_top2_kernel(const float* logits, int ld, int vocab,
                                                                    int* out_id, float* out_margin) {
    __shared__ Best sh_best[32];
    const float* lg = logits + (size_t)blockIdx.x * ld;
    Best b{-INFINITY, 0xffffffffu};
    for (uint32_t i = threadIdx.x; i < (uint32_t)vocab; i += kSampThreads)
        if (ranks_before(lg[i], i, b.v, b.i)) { b.v = lg[i]; b.i = i; }
    b = block_best(b, sh_best);
    Best s{-INFINITY, 0xffffffffu};
    for (uint32_t i = threadIdx.x; i < (uint32_t)vocab; i += kSampThreads)
        if (i != b.i && ranks_before(lg[i], i, s.v, s.i)) { s.v = lg[i]; s.i = i; }
    s = block_best(s, sh_best);
    if (threadIdx.x == 0) { out_id[blockIdx.x] = (int)b.i; if (out_margin) out_margin[blockIdx.x] = b.v - s.v; }
}

}  // namespace ps

PS_API int ps_sample(const void* logits, int ld, int vocab, int rows, const void* params, const void* mask,
                     int mask_words, const void* mask_active, void* out, void* status, cudaStream_t stream) {
    using namespace ps;
    if (rows <= 0 || vocab <= 0) return (int)cudaErrorInvalidValue;
    SampleArgs a;
    a.logits = (const float*)logits; a.ld = ld; a.vocab = vocab; a.rows = rows;
    a.params = (const SamplingRow*)params; a.mask = (const uint32_t*)mask; a.mask_words = mask_words;
    a.mask_active = (const uint8_t*)mask_active; a.out = (int*)out; a.status = (uint32_t*)status;
    sample_kernel<<<rows, kSampThreads, 0, stream>>>(a);
    return PS_LAUNCH_CHECK();
}

PS_API int ps_argmax_top2(const void* logits, int ld, int vocab, int rows, void* out_id, void* out_margin,
                          cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return (int)cudaErrorInvalidValue;
    ps::argmax_top2_kernel<<<rows, ps::kSampThreads, 0, stream>>>((const float*)logits, ld, vocab, (int*)out_id,
                                                                    (float*)out_margin);
    return PS_LAUNCH_CHECK();
}
