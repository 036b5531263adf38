// Expand a tiled weight matrix (BF16 / NVFP4 / MXFP8, layout in gemv_core.cuh) into a row-major bf16
// scratch matrix [N, ldo] for the tensor-core prefill GEMM.  Pure streaming: reads 0.56-2 B/weight,
// writes 2 B/weight; at prefill row counts this is a few percent of the GEMM it feeds.
// The scaling applied is exactly decode's: w = code * block_scale * tensor_scale, rounded once to bf16.
#include "gemv_core.cuh"

namespace ps {

template <int WF>
__global__ void dequant_tiled_kernel(const uint8_t* __restrict__ w, int N, int K, float gscale,
                                     __nv_bfloat16* __restrict__ out, int ldo) {
    constexpr int CH = WTraits<WF>::kChunk;
    constexpr int kBlock = WTraits<WF>::kBlockBytes;
    const int steps = gemv_steps<WF>(K);
    const int n_quads = (N + 3) / 4;
    // one warp per (quad, step) block, lane = 16-byte chunk, loop over the 4 rows
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n_quads * steps) return;
    const int lane = threadIdx.x & 31;
    const int q = (int)(unit / steps), st = (int)(unit % steps);
    const uint8_t* blk = w + (size_t)unit * kBlock;
    const int k = (st * 32 + lane) * CH;
    if (k >= K) return;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int n = q * 4 + r;
        if (n >= N) break;
        const uint4 c = *reinterpret_cast<const uint4*>(blk + r * 512 + lane * 16);
        __nv_bfloat16* o = out + (size_t)n * ldo + k;
        if constexpr (WF == W_BF16) {
            *reinterpret_cast<uint4*>(o) = c;
        } else if constexpr (WF == W_NVFP4) {
            uint32_t sh[2];
            cvt_e4m3x4(*reinterpret_cast<const uint16_t*>(blk + 2048 + r * 64 + lane * 2), sh);
            const float2 sc = __half22float2(as_half2(sh[0]));
            const uint32_t wq[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t h[4];
                cvt_e2m1x8(wq[j], h);
                const float s = (j < 2 ? sc.x : sc.y) * gscale;
                uint32_t ob[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(as_half2(h[i]));
                    ob[i] = f32x2_to_bf16x2_bits(f.x * s, f.y * s);
                }
                *reinterpret_cast<uint4*>(o + j * 8) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
            }
        } else {
            const float s = __uint_as_float((uint32_t)blk[2048 + r * 16 + (lane >> 1)] << 23) * gscale;
            const uint32_t wq[4] = {c.x, c.y, c.z, c.w};
            uint32_t ob[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t h[2];
                cvt_e4m3x4(wq[j], h);
                const float2 f0 = __half22float2(as_half2(h[0])), f1 = __half22float2(as_half2(h[1]));
                ob[2 * j] = f32x2_to_bf16x2_bits(f0.x * s, f0.y * s);
                ob[2 * j + 1] = f32x2_to_bf16x2_bits(f1.x * s, f1.y * s);
            }
            *reinterpret_cast<uint4*>(o) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
            *reinterpret_cast<uint4*>(o + 8) = make_uint4(ob[4], ob[5], ob[6], ob[7]);
        }
    }
}

}  // namespace ps

PS_API int ps_dequant_tiled(int wfmt, const void* w_tiled, int N, int K, float gscale, void* out, int ldo,
                            cudaStream_t stream) {
    using namespace ps;
    if (N <= 0 || K <= 0 || (K % 32) || (ldo % 8)) return (int)cudaErrorInvalidValue;
    const int n_quads = (N + 3) / 4;
    long long units;
    const int wpb = 8;
    switch (wfmt) {
        case W_BF16:
            units = (long long)n_quads * gemv_steps<W_BF16>(K);
            dequant_tiled_kernel<W_BF16><<<(unsigned)((units + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
                (const uint8_t*)w_tiled, N, K, gscale, (__nv_bfloat16*)out, ldo);
            break;
        case W_NVFP4:
            units = (long long)n_quads * gemv_steps<W_NVFP4>(K);
            dequant_tiled_kernel<W_NVFP4><<<(unsigned)((units + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
                (const uint8_t*)w_tiled, N, K, gscale, (__nv_bfloat16*)out, ldo);
            break;
        case W_MXFP8:
            units = (long long)n_quads * gemv_steps<W_MXFP8>(K);
            dequant_tiled_kernel<W_MXFP8><<<(unsigned)((units + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
                (const uint8_t*)w_tiled, N, K, gscale, (__nv_bfloat16*)out, ldo);
            break;
        default: return (int)cudaErrorInvalidValue;
    }
    return PS_LAUNCH_CHECK();
}
