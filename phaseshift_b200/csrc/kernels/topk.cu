// Exact top-k (k <= 128) over a logits row by radix select: four 8-bit passes over order-preserving
// integer keys find the k-th largest value exactly, one more sweep collects the winners (ties at the
// threshold are resolved towards the lower token id), and a bitonic sort orders the k survivors.  One CTA
// of 1024 threads per row; the row is read five times from L2/HBM (600 KB at vocab 151936).
// Used for the drafter's candidate sets and available as the active-set primitive for top-k sampling;
// counterpart of the reference's radix_topn / coarse_topn kernels
// (src/phaseshift/models/qwen35/kernels/dflash2/radix_topn.hip:41-384, topk_optimized.hip:95-242).
#include "ps_common.cuh"

namespace ps {

constexpr int kTopkThreads = 1024;
constexpr int kTopkMax = 128;

__device__ __forceinline__ uint32_t ordered_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);       // larger float <=> larger key; NaNs sort to the ends
}

__device__ __forceinline__ bool tk_allowed(const uint32_t* m, uint32_t tok) {
    return m == nullptr || ((m[tok >> 5] >> (tok & 31u)) & 1u);
}

__global__ void __launch_bounds__(kTopkThreads) topk_kernel(const float* __restrict__ logits, long long ld, int vocab, int k,
                                                             const uint32_t* __restrict__ mask, int mask_words,
                                                             int* __restrict__ out_ids, float* __restrict__ out_vals) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_need, s_cnt_gt, s_cnt_eq, s_fill, s_run;
    __shared__ uint32_t s_warp[32];
    __shared__ float s_val[kTopkMax];
    __shared__ int s_id[kTopkMax];
    const float* lg = logits + (long long)blockIdx.x * ld;
    const uint32_t* m = mask != nullptr ? mask + (long long)blockIdx.x * mask_words : nullptr;
    const int t = threadIdx.x;
    if (t == 0) { s_prefix = 0; s_need = (uint32_t)k; s_fill = 0; s_run = 0; }
    // ---- four radix passes, most significant byte first
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (t < 256) hist[t] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const uint32_t pmask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = t; i < vocab; i += kTopkThreads) {
            if (!tk_allowed(m, i)) continue;
            const uint32_t key = ordered_key(lg[i]);
            if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
        }
        __syncthreads();
        if (t == 0) {
            uint32_t need = s_need, b = 255;
            for (;; --b) {                      // walk from the largest byte value down
                if (hist[b] >= need || b == 0) break;
                need -= hist[b];
            }
            s_prefix = prefix | (b << shift);
            s_need = hist[b] >= need ? need : hist[b];   // fewer allowed tokens than k: take what exists
        }
        __syncthreads();
    }
    const uint32_t T = s_prefix;                 // key of the k-th largest allowed element
    // ---- count and collect everything strictly above the threshold
    if (t == 0) { s_cnt_gt = 0; s_cnt_eq = 0; }
    __syncthreads();
    for (int i = t; i < vocab; i += kTopkThreads) {
        if (!tk_allowed(m, i)) continue;
        const uint32_t key = ordered_key(lg[i]);
        if (key > T) {
            const uint32_t slot = atomicAdd(&s_fill, 1u);
            if (slot < (uint32_t)k) { s_val[slot] = lg[i]; s_id[slot] = i; }
            atomicAdd(&s_cnt_gt, 1u);
        } else if (key == T) {
            atomicAdd(&s_cnt_eq, 1u);
        }
    }
    __syncthreads();
    const uint32_t n_gt = min(s_cnt_gt, (uint32_t)k);
    const uint32_t want_eq = min((uint32_t)k - n_gt, s_cnt_eq);
    // ---- threshold ties: the lowest ids win; sweep in id order with a block-wide running count
    if (want_eq > 0) {
        for (int base = 0; base < vocab && s_run < want_eq; base += kTopkThreads) {
            const int i = base + t;
            const bool hit = i < vocab && tk_allowed(m, i) && ordered_key(lg[i]) == T;
            const uint32_t bal = __ballot_sync(0xffffffffu, hit);
            const int lane = t & 31, wp = t >> 5;
            if (lane == 0) s_warp[wp] = __popc(bal);
            __syncthreads();
            uint32_t before = s_run;
            for (int w2 = 0; w2 < wp; ++w2) before += s_warp[w2];
            const uint32_t pos = before + __popc(bal & ((1u << lane) - 1u));
            if (hit && pos < want_eq) { s_val[n_gt + pos] = lg[i]; s_id[n_gt + pos] = i; }
            __syncthreads();
            if (t == 0) { uint32_t tot = 0; for (int w2 = 0; w2 < 32; ++w2) tot += s_warp[w2]; s_run += tot; }
            __syncthreads();
        }
    }
    const int found = (int)(n_gt + want_eq);
    // ---- bitonic sort of the survivors (descending value, ascending id on ties), padded to 128
    for (int i = t; i < kTopkMax; i += kTopkThreads) if (i >= found) { s_val[i] = -INFINITY; s_id[i] = 0x7fffffff; }
    __syncthreads();
    for (int size = 2; size <= kTopkMax; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (t < kTopkMax) {
                const int j = t ^ stride;
                if (j > t) {
                    const bool desc = (t & size) == 0;
                    const float va = s_val[t], vb = s_val[j];
                    const int ia = s_id[t], ib = s_id[j];
                    const bool a_first = va > vb || (va == vb && ia < ib);      // a ranks before b
                    if (desc ? !a_first : a_first) { s_val[t] = vb; s_val[j] = va; s_id[t] = ib; s_id[j] = ia; }
                }
            }
            __syncthreads();
        }
    }
    for (int i = t; i < k; i += kTopkThreads) {
        out_ids[(long long)blockIdx.x * k + i] = i < found ? s_id[i] : -1;
        out_vals[(long long)blockIdx.x * k + i] = i < found ? s_val[i] : -INFINITY;
    }
}

}  // namespace ps

// ids / vals: [rows, k]; rows with fewer than k allowed tokens are padded with id -1 / -inf.
PS_API int ps_topk(const void* logits, long long ld, int vocab, int rows, int k, const void* mask, int mask_words, void* out_ids,
                   void* out_vals, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0 || k < 1 || k > ps::kTopkMax) return (int)cudaErrorInvalidValue;
    ps::topk_kernel<<<rows, ps::kTopkThreads, 0, stream>>>((const float*)logits, ld, vocab, k, (const uint32_t*)mask, mask_words,
                                                           (int*)out_ids, (float*)out_vals);
    return PS_LAUNCH_CHECK();
}
