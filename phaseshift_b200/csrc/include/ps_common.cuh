// Shared device/host helpers for every phaseshift_b200 CUDA kernel (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

#define PS_API extern "C" __attribute__((visibility("default")))

// Status codes written to a device status word by kernels that can fail at run time
// (bounded waits, invalid page ids).  Mirrors the reference's ProgramStatus idea
// (include/phaseshift/runtime/program/device_program.h:7-51): hosts read the word
// after the step and poison the affected sequences instead of trapping the GPU.
enum PsDeviceStatus : uint32_t {
    PS_DEV_OK = 0,
    PS_DEV_BAD_INDEX = 1,      // page / slot / row index out of range; the access was skipped
    PS_DEV_WAIT_TIMEOUT = 2,   // a bounded spin-wait (peer flag, mbarrier) ran out of budget
    PS_DEV_SAMPLING_FAILED = 3,
    PS_DEV_NONFINITE = 4,
    PS_DEV_CHECK_FAILED = 5,   // checked build only: a descriptor / row / slot assertion failed; the block returned
};

// Budget, in GPU clock cycles, of every bounded device-side wait (mbarrier, peer flag, stream-K flag).
// One definition for the whole library (elementwise.cu); ps_set_wait_budget() changes it, launchers pass
// the current value to their kernels.  The default is about one second at B200 clocks.
extern long long g_ps_wait_budget_cycles;

// Checked build (-DPS_CHECKED, a second library beside the normal one; the stand-in for a device sanitizer): kernels
// validate the descriptors they are handed -- slots, row ranges -- against limits the host registers once per
// translation unit, report PS_DEV_CHECK_FAILED through the registered status word and return instead of touching
// memory.  PS_CHECK conditions must be uniform over the thread block (they guard an early return).
#ifdef PS_CHECKED
namespace ps {
struct Limits { int max_slots, max_rows; uint32_t* status; };
static __device__ Limits g_limits = {1 << 30, 1 << 30, nullptr};
}
#define PS_DEFINE_LIMITS_SETTER(tag)                                                                   \
    PS_API int ps_set_limits_##tag(int max_slots, int max_rows, void* status) {                        \
        ps::Limits l{max_slots, max_rows, (uint32_t*)status};                                          \
        return (int)cudaMemcpyToSymbol(ps::g_limits, &l, sizeof(l));                                   \
    }
#define PS_CHECK(cond)                                                                                 \
    do {                                                                                               \
        if (!(cond)) {                                                                                 \
            if (ps::g_limits.status != nullptr) atomicCAS(ps::g_limits.status, 0u, (uint32_t)PS_DEV_CHECK_FAILED); \
            return;                                                                                    \
        }                                                                                              \
    } while (0)
#define PS_SLOT_OK(s) ((s) >= 0 && (s) < ps::g_limits.max_slots)
#define PS_ROWS_OK(r0, n) ((r0) >= 0 && (n) >= 0 && (r0) + (n) <= ps::g_limits.max_rows)
#else
#define PS_DEFINE_LIMITS_SETTER(tag)
#define PS_CHECK(cond) ((void)0)
#define PS_SLOT_OK(s) true
#define PS_ROWS_OK(r0, n) true
#endif

// Launch helpers return the CUDA error code as int (0 = cudaSuccess).
#define PS_LAUNCH_CHECK() (int)cudaGetLastError()

namespace ps {

constexpr int kWarp = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum for blockDim.x <= 1024; `red` is >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? red[lane] : -3.4e38f;
    r = warp_max(r);
    return r;
}

// Fused block reduction of N sums (and optionally one max) with two barriers in total.
// `red` needs 32 * (N + 1) floats.  Every thread receives all results.
template <int N>
__device__ __forceinline__ void block_sum_n(float (&v)[N], float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = warp_sum(v[i]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < N; ++i) red[i * 32 + w] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = warp_sum(lane < nw ? red[i * 32 + lane] : 0.f);
}
__device__ __forceinline__ void block_sum_max(float& s, float& m, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    s = warp_sum(s); m = warp_max(m);
    __syncthreads();
    if (lane == 0) { red[w] = s; red[32 + w] = m; }
    __syncthreads();
    s = warp_sum(lane < nw ? red[lane] : 0.f);
    m = warp_max(lane < nw ? red[32 + lane] : -3.4e38f);
}

__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float2 bf16x2_bits_to_f32x2(uint32_t u) {
    float2 r;
    r.x = __uint_as_float(u << 16);
    r.y = __uint_as_float(u & 0xffff0000u);
    return r;
}
__device__ __forceinline__ uint32_t f32x2_to_bf16x2_bits(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// UE4M3 / E4M3 byte -> float (finite values only; 0x7f/0xff decode as NaN per OCP).
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&hr));
}
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code) {
    if (status != nullptr) atomicCAS(status, 0u, code);
}

// Launch with programmatic dependent launch allowed: the kernel may be scheduled while its stream
// predecessor is still draining; it must call cudaGridDependencySynchronize() before touching anything
// the predecessor wrote.  PS_PDL=0 in the environment turns the attribute off.
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("PS_PDL"); v = (e == nullptr || e[0] != '0') ? 1 : 0; }
    return v != 0;
}
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace ps
