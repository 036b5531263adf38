// Sampling contract shared by host (C++ runtime, tests) and device (sampling.cu).
//
// Behavioural contract follows the reference (docs/developer/sampling.md:35-213):
//   * mode 0 = none, 1 = greedy (argmax, ties -> lower token id), 2 = stochastic (Gumbel-max);
//   * randomness is a counter hash of (seed, sample_index, attempt, token_id) only, so batch
//     placement, prefix-cache hits and chunking never change a sample; host and device agree bit
//     for bit on the uniform;
//   * top-k / top-p are membership tests on the full softmax: a Gumbel-max candidate c is accepted
//     iff fewer than top_k tokens rank before it and the probability mass ranking before it is
//     below top_p * Z; otherwise the draw is repeated with attempt+1 (at most kMaxAttempts);
//   * a constraint bitmask (1 bit per token, 32 tokens per word) removes tokens before everything.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define PS_HD __host__ __device__ __forceinline__
#else
#define PS_HD inline
#endif

namespace ps {

constexpr uint32_t kSamplingNone = 0u, kSamplingGreedy = 1u, kSamplingStochastic = 2u;
constexpr uint32_t kMaxSamplingAttempts = 4096u;

struct SamplingRow {      // one per output row, uploaded with the batch
    uint32_t mode;
    float temperature;
    float top_p;
    uint32_t top_k;
    uint64_t seed;
    uint64_t sample_index;   // number of tokens the request has generated so far
};

PS_HD uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Counter-based generator: four chained SplitMix64 finalisers, one per key component.
PS_HD uint32_t sampling_bits(uint64_t seed, uint64_t sample_index, uint64_t attempt, uint64_t token_id) {
    uint64_t h = mix64(seed ^ 0x6A09E667F3BCC908ull);
    h = mix64(h + sample_index * 0xD6E8FEB86659FD93ull);
    h = mix64(h + attempt * 0xA0761D6478BD642Full);
    h = mix64(h + token_id * 0xE7037ED1A0B428DBull);
    return (uint32_t)(h >> 32);
}

// Uniform strictly inside (0,1): (top 23 bits + 0.5) * 2^-23, exact in fp32 so neither 0 nor 1 can
// appear (a (bits+0.5)*2^-32 form rounds to 1.0 for the top 128 counter values and makes the Gumbel
// noise infinite).
PS_HD float sampling_uniform(uint64_t seed, uint64_t sample_index, uint64_t attempt, uint64_t token_id) {
    return ((float)(sampling_bits(seed, sample_index, attempt, token_id) >> 9) + 0.5f) * (1.0f / 8388608.0f);
}

PS_HD bool ranks_before(float va, uint32_t ia, float vb, uint32_t ib) {
    return va > vb || (va == vb && ia < ib);
}

}  // namespace ps
