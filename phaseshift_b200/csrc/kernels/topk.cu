// Exact top-k (k <= 128) over fp32 logits rows, sorted (value descending, token id ascending on ties).
// Two launches that keep every SM busy even for a handful of rows:
//   1. the row is cut into chunks; one CTA per (chunk, row) holds its chunk in registers as 64-bit keys
//      (order-preserving value bits | inverted token id) and extracts its k largest by k block-wide arg-max rounds;
//   2. one CTA per row extracts the k largest of the chunks' winners the same way.
// A 64-bit key compares like (value, lower id first), so ties need no second criterion and the result is exact.
// The row is read once.  Used for the drafter's candidate sets and as the active-set primitive for top-k
// sampling; counterpart of the reference's radix_topn / coarse_topn kernels
// (src/phaseshift/models/qwen35/kernels/dflash2/radix_topn.hip:41-384, topk_optimized.hip:95-242).
#include "ps_common.cuh"

namespace ps {

constexpr int kTopkMax = 128;
constexpr int kTopkChunkThreads = 256, kTopkMergeThreads = 1024, kTopkRegs = 16;
constexpr int kTopkMaxChunks = 128;

__device__ __forceinline__ unsigned long long topk_key(float v, uint32_t id) {
    v += 0.0f;                                                   // -0.0 ranks with +0.0
    const uint32_t u = __float_as_uint(v);
    const uint32_t k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float <=> larger key
    return ((unsigned long long)k << 32) | (unsigned long long)(0xffffffffu - id);
}

__device__ __forceinline__ bool tk_allowed(const uint32_t* m, uint32_t tok) {
    return m == nullptr || ((m[tok >> 5] >> (tok & 31u)) & 1u);
}

// k rounds of: block-wide maximum of the live keys, the owner retires its key, thread 0 records the winner.
template <int THREADS>
__device__ __forceinline__ void topk_rounds(unsigned long long (&keys)[kTopkRegs], int k, unsigned long long* out,
                                            unsigned long long* s_red) {
    constexpr int WARPS = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int it = 0; it < k; ++it) {
        unsigned long long best = 0;
#pragma unroll
        for (int e = 0; e < kTopkRegs; ++e) best = keys[e] > best ? keys[e] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) s_red[warp] = best;
        __syncthreads();
        if (warp == 0) {                                            // second level: one warp, one shared result
            unsigned long long v = lane < WARPS ? s_red[lane] : 0ull;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
                v = other > v ? other : v;
            }
            if (lane == 0) s_red[WARPS] = v;
        }
        __syncthreads();
        const unsigned long long w = s_red[WARPS];
        if (w != 0) {
#pragma unroll
            for (int e = 0; e < kTopkRegs; ++e) if (keys[e] == w) keys[e] = 0;
        }
        if (threadIdx.x == 0) out[it] = w;
    }
}

__global__ void __launch_bounds__(kTopkChunkThreads) topk_chunk_kernel(const float* __restrict__ logits, long long ld, int vocab, int k,
                                                                       int chunk, const uint32_t* __restrict__ mask, int mask_words,
                                                                       unsigned long long* __restrict__ ws) {
    __shared__ unsigned long long s_red[kTopkChunkThreads / 32 + 1];
    const int row = blockIdx.y, c = blockIdx.x;
    const float* lg = logits + (long long)row * ld;
    const uint32_t* m = mask != nullptr ? mask + (long long)row * mask_words : nullptr;
    unsigned long long keys[kTopkRegs];
    const int lo = c * chunk, hi = min(vocab, lo + chunk);
#pragma unroll
    for (int e = 0; e < kTopkRegs; ++e) {
        const int i = lo + threadIdx.x + e * kTopkChunkThreads;
        keys[e] = (i < hi && tk_allowed(m, (uint32_t)i)) ? topk_key(lg[i], (uint32_t)i) : 0ull;
    }
    topk_rounds<kTopkChunkThreads>(keys, k, ws + ((long long)row * gridDim.x + c) * k, s_red);
}

__global__ void __launch_bounds__(kTopkMergeThreads) topk_merge_kernel(const unsigned long long* __restrict__ ws, int n_cand, int k,
                                                                       int* __restrict__ out_ids, float* __restrict__ out_vals) {
    __shared__ unsigned long long s_red[kTopkMergeThreads / 32 + 1];
    __shared__ unsigned long long s_out[kTopkMax];
    const int row = blockIdx.x;
    unsigned long long keys[kTopkRegs];
#pragma unroll
    for (int e = 0; e < kTopkRegs; ++e) {
        const int i = threadIdx.x + e * kTopkMergeThreads;
        keys[e] = i < n_cand ? ws[(long long)row * n_cand + i] : 0ull;
    }
    topk_rounds<kTopkMergeThreads>(keys, k, s_out, s_red);
    __syncthreads();
    for (int i = threadIdx.x; i < k; i += kTopkMergeThreads) {
        const unsigned long long w = s_out[i];
        const uint32_t kk = (uint32_t)(w >> 32);
        const uint32_t u = (kk & 0x80000000u) ? (kk & 0x7fffffffu) : ~kk;
        out_ids[(long long)row * k + i] = w != 0 ? (int)(0xffffffffu - (uint32_t)w) : -1;
        out_vals[(long long)row * k + i] = w != 0 ? __uint_as_float(u) : -INFINITY;
    }
}

}  // namespace ps

// Workspace bytes ps_topk needs for `rows` rows of `vocab` logits and this k.
PS_API long long ps_topk_workspace_bytes(int vocab, int rows, int k) {
    const int chunks = (vocab + 2047) / 2048;
    return (long long)rows * (chunks < 1 ? 1 : chunks) * k * 8;
}

// ids / vals: [rows, k]; rows with fewer than k allowed tokens are padded with id -1 / -inf.
PS_API int ps_topk(const void* logits, long long ld, int vocab, int rows, int k, const void* mask, int mask_words, void* out_ids,
                   void* out_vals, void* ws, long long ws_bytes, cudaStream_t stream) {
    using namespace ps;
    if (rows <= 0 || vocab <= 0 || k < 1 || k > kTopkMax || ws == nullptr) return (int)cudaErrorInvalidValue;
    int chunks = (vocab + 2047) / 2048;                               // ~8 keys per thread
    if (chunks > kTopkMaxChunks) return (int)cudaErrorInvalidValue;  // vocab beyond 262144: not a language-model head
    const int chunk = (vocab + chunks - 1) / chunks;
    if (chunk > kTopkChunkThreads * kTopkRegs || chunks * k > kTopkMergeThreads * kTopkRegs) return (int)cudaErrorInvalidValue;
    if (ws_bytes < (long long)rows * chunks * k * 8) return (int)cudaErrorInvalidValue;
    topk_chunk_kernel<<<dim3(chunks, rows), kTopkChunkThreads, 0, stream>>>((const float*)logits, ld, vocab, k, chunk, (const uint32_t*)mask,
                                                                           mask_words, (unsigned long long*)ws);
    topk_merge_kernel<<<rows, kTopkMergeThreads, 0, stream>>>((const unsigned long long*)ws, chunks * k, k, (int*)out_ids, (float*)out_vals);
    return PS_LAUNCH_CHECK();
}
