// NVFP4 key/value pages: the 4-bit storage format of the paged cache.
//
// One cached row (a token of one KV head, D values) is stored as
//     [ D/2 code bytes | D/16 block-scale bytes | padding to a multiple of 16 bytes ]
// where byte j of the codes holds the E2M1 values 2j (low nibble) and 2j+1 (high nibble), and block-scale byte b
// is the UE4M3 scale of values 16b .. 16b+15.  A third, fp32 factor per (page, head, token) lives in the pools'
// scale arrays (the same arrays the FP8 pools use):
//     value = e2m1(code) * ue4m3(block scale) * token scale,     token scale = max|row| / (6 * 448).
// 4.5 bits per value plus 4 bytes per row: 148 bytes for a 256-wide head against 512 in bf16 and 260 in FP8.
//
// Counterpart of the reference's 4-bit KV block codec (include/phaseshift/quantization/psq/psq4_kv.h:1-79: 32-value
// blocks, codebook codes, one bf16 scale per block); here the codes are the hardware's E2M1 and the scales two-level,
// so conversion is one `cvt` per pair of values.
#pragma once
#include <cuda_fp4.h>

#include "ps_common.cuh"

namespace ps {

__host__ __device__ inline int kv_fp4_row_bytes(int D) { return ((D / 2 + D / 16) + 15) & ~15; }

__device__ __forceinline__ float kv_fp4_token_scale(float amax) { return amax > 0.f ? amax * (1.f / (6.f * 448.f)) : 1.f; }

// 16 values -> 8 code bytes + one block-scale byte.  `ts` = the row's token scale.
__device__ __forceinline__ void kv_fp4_quant16(const float* v, float ts, uint2& codes, uint8_t& sf) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    sf = f32_to_e4m3(__fdiv_rn(amax, __fmul_rn(6.f, ts)));
    const float sf_f = e4m3_to_f32(sf);
    const float inv = sf_f > 0.f ? __fdiv_rn(1.f, __fmul_rn(sf_f, ts)) : 0.f;
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t acc = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 pr = make_float2(__fmul_rn(v[h * 8 + 2 * j], inv), __fmul_rn(v[h * 8 + 2 * j + 1], inv));
            acc |= (uint32_t)__nv_cvt_float2_to_fp4x2(pr, __NV_E2M1, cudaRoundNearest) << (8 * j);
        }
        w[h] = acc;
    }
    codes = make_uint2(w[0], w[1]);
}

// One code byte (two values) times a block scale -> two bf16 values (exact: at most six significant bits).
__device__ __forceinline__ uint32_t kv_fp4_byte_to_bf16x2(uint32_t byte, float sf_f) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xffu), __NV_E2M1);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    return f32x2_to_bf16x2_bits(f.x * sf_f, f.y * sf_f);
}

// 16 code bytes (32 values, two blocks) with their two block scales -> 32 bf16 values as four 16-byte words.
__device__ __forceinline__ void kv_fp4_piece_to_bf16(const uint4& c, uint32_t two_scales, uint4 (&out)[4]) {
    const float s0 = e4m3_to_f32((uint8_t)(two_scales & 0xffu)), s1 = e4m3_to_f32((uint8_t)((two_scales >> 8) & 0xffu));
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = kv_fp4_byte_to_bf16x2(w[j >> 2] >> ((j & 3) * 8), j < 8 ? s0 : s1);
#pragma unroll
    for (int q = 0; q < 4; ++q) out[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
}

}  // namespace ps
