// Stand-alone all-reduce over NVLink peer memory for prefill-sized activations (more rows than the
// fused combine in the projection epilogue handles): out = sum over ranks of partial [rows, n] (bf16)
// + residual, written as bf16.  Two variants:
//
//   * peer one-shot : every rank waits (bounded) until the same CTA of every peer has started -- which, by
//     stream order on the peer, means the peer's partial is complete in its symmetric buffer -- then
//     reads all `size` partials with plain peer loads and adds them in rank order 0..size-1 in fp32, so
//     every rank holds bit-identical sums.  One launch, one barrier, no second pass.
//   * multimem two-shot : rank r reduces the 16-byte chunks with (chunk % size == r) through the
//     NVSwitch (`multimem.ld_reduce`, fp32 accumulation) and broadcasts them with `multimem.st` into
//     every rank's result buffer; after a second barrier each rank adds the residual from its local
//     copy.  Every element is reduced exactly once, so ranks agree bit for bit, and each GPU moves only
//     1/size of the data through its links twice.
//
// Inputs are double-buffered by the parity of a per-CTA collective counter: a rank can be at most one
// collective ahead of its slowest peer, so a buffer is rewritten only after every peer has finished
// reading it.  Every wait is bounded by a clock budget and reports PS_DEV_WAIT_TIMEOUT through the status
// word instead of hanging.  The reference's transport does leader-reduce + broadcast with a host
// rendezvous per collective (src/phaseshift/runtime/tp/hip_peer_tp_transport.hip:314-369).
#include "ps_common.cuh"

namespace ps {

constexpr int kArMaxRanks = 8;

struct ArArgs {
    int size, rank;
    const __nv_bfloat16* in[kArMaxRanks];   // every rank's partial for this parity (peer pointers), dense [rows, n]
    __nv_bfloat16* mc_in;                   // multicast address of the same buffer (multimem variant), else null
    __nv_bfloat16* mc_res;                  // multicast address of the result buffer (multimem variant)
    const __nv_bfloat16* res_local;         // local address of the result buffer (multimem variant)
    uint32_t* flags[kArMaxRanks];           // rank r's flags: [2][grid][size]
    uint32_t* counter;                      // local [grid]
    const __nv_bfloat16* residual; int ld_res;
    __nv_bfloat16* out; int ldo;
    int rows, n;
    uint32_t* status;
};

// Signal every peer and wait for every peer at (phase, this CTA).  Returns false on timeout.
__device__ __forceinline__ bool peer_barrier(uint32_t* const* flags, int size, int rank, int phase, uint32_t val, bool* s_fail,
                                             long long budget) {
    __syncthreads();
    if (threadIdx.x < size) {
        __threadfence_system();
        const size_t base = ((size_t)phase * gridDim.x + blockIdx.x) * size;
        uint32_t* f = flags[threadIdx.x] + base + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(val) : "memory");
        const uint32_t* mine = flags[rank] + base + threadIdx.x;
        const long long t0 = clock64();
        uint32_t seen;
        do {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int32_t)(seen - val) >= 0) break;
            if (clock64() - t0 > budget) { *s_fail = true; break; }
        } while (true);
    }
    __syncthreads();
    return !*s_fail;
}
__device__ __forceinline__ bool ar_barrier(const ArArgs& a, int phase, uint32_t val, bool* s_fail, long long budget) {
    return peer_barrier(a.flags, a.size, a.rank, phase, val, s_fail, budget);
}

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = bf16x2_bits_to_f32x2(w[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
}

__device__ __forceinline__ void finish_chunk(const ArArgs& a, long long chunk, float (&acc)[8]) {
    const int per_row = a.n >> 3;
    const int row = (int)(chunk / per_row), col = (int)(chunk % per_row) << 3;
    if (a.residual != nullptr) {
        // the sum is rounded to bf16 before the residual add, like projection-then-add
        const uint4 r = *reinterpret_cast<const uint4*>(a.residual + (size_t)row * a.ld_res + col);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = bf16x2_bits_to_f32x2(w[i]);
            acc[2 * i] = bf16_to_f32(f32_to_bf16(acc[2 * i])) + f.x;
            acc[2 * i + 1] = bf16_to_f32(f32_to_bf16(acc[2 * i + 1])) + f.y;
        }
    }
    *reinterpret_cast<uint4*>(a.out + (size_t)row * a.ldo + col) =
        make_uint4(f32x2_to_bf16x2_bits(acc[0], acc[1]), f32x2_to_bf16x2_bits(acc[2], acc[3]),
                   f32x2_to_bf16x2_bits(acc[4], acc[5]), f32x2_to_bf16x2_bits(acc[6], acc[7]));
}

__global__ void __launch_bounds__(256) allreduce_peer_kernel(const ArArgs a, const long long budget) {
    __shared__ bool s_fail;
    __shared__ uint32_t s_val;
    if (threadIdx.x == 0) { s_fail = false; s_val = a.counter[blockIdx.x] + 1u; }
    __syncthreads();
    const uint32_t val = s_val;
    if (!ar_barrier(a, 0, val, &s_fail, budget)) { if (threadIdx.x == 0) set_status(a.status, PS_DEV_WAIT_TIMEOUT); return; }
    if (threadIdx.x == 0) a.counter[blockIdx.x] = val;
    const long long chunks = (long long)a.rows * (a.n >> 3);
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (long long)gridDim.x * blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < a.size; ++r) acc_bf16x8(acc, __ldcv(reinterpret_cast<const uint4*>(a.in[r]) + c));
        finish_chunk(a, c, acc);
    }
}

__global__ void __launch_bounds__(256) allreduce_multimem_kernel(const ArArgs a, const long long budget) {
    __shared__ bool s_fail;
    __shared__ uint32_t s_val;
    if (threadIdx.x == 0) { s_fail = false; s_val = a.counter[blockIdx.x] + 1u; }
    __syncthreads();
    const uint32_t val = s_val;
    if (!ar_barrier(a, 0, val, &s_fail, budget)) { if (threadIdx.x == 0) set_status(a.status, PS_DEV_WAIT_TIMEOUT); return; }
    const long long chunks = (long long)a.rows * (a.n >> 3);
    const long long stride = (long long)gridDim.x * blockDim.x;
    // shot 1: reduce my share through the switch and broadcast it into every rank's result buffer
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i * a.size + a.rank < chunks; i += stride) {
        const long long c = i * a.size + a.rank;
        uint32_t x, y, z, w;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(reinterpret_cast<const uint4*>(a.mc_in) + c) : "memory");
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                     ::"l"(reinterpret_cast<uint4*>(a.mc_res) + c), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
    }
    if (!ar_barrier(a, 1, val, &s_fail, budget)) { if (threadIdx.x == 0) set_status(a.status, PS_DEV_WAIT_TIMEOUT); return; }
    if (threadIdx.x == 0) a.counter[blockIdx.x] = val;
    // shot 2: the CTA with the same index on rank (c % size) produced chunk c; read the local copy
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i * a.size < chunks; i += stride) {
        for (int r = 0; r < a.size; ++r) {
            const long long c = i * a.size + r;
            if (c >= chunks) break;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            acc_bf16x8(acc, __ldcv(reinterpret_cast<const uint4*>(a.res_local) + c));
            finish_chunk(a, c, acc);
        }
    }
}

// ---- second half of the fused row-parallel projection for many rows: reduce + residual + all-gather.
// The projection kernels of all ranks have pushed their bf16 partials of MY rows into my receive buffer
// ([source rank][rpr][ld]; csrc/kernels/gemm_bs.cu, TpScatter) -- or, for projection kernels that cannot push, left
// their whole partial in symmetric memory, from where the owner pulls its rows (two-shot all-reduce).  Barrier A (the same CTA of every peer has started, so
// by stream order its projection -- and with it its pushes -- is complete), then every rank adds the partials of the
// rows it owns in rank order, rounds, adds the residual and stores the finished rows into EVERY rank's output buffer
// (16-byte peer stores); barrier B (every peer's stores into my output are complete, and every peer is done reading
// its receive buffer, so the next projection may push again).  Each row is reduced exactly once: ranks agree bit for bit.
struct RgArgs {
    int size, rank, rows, n, rpr;
    // Where the partials of my rows are: source r's rows start at src[r], row (m - src_row0) of pitch ld.
    //  push form: src[r] = my receive buffer + r * rpr * ld, src_row0 = my first row (local loads)
    //  pull form: src[r] = rank r's partial [rows, ld] in symmetric memory, src_row0 = 0 (peer loads of my rows only)
    const __nv_bfloat16* src[kArMaxRanks]; int src_row0, ld;
    // optional first phase (projection kernels that cannot push themselves): my whole partial [rows, ld_partial] is
    // dealt to the owners' receive buffers by this kernel (remote STORES only; nothing waits on a remote load)
    const __nv_bfloat16* partial; int ld_partial;
    __nv_bfloat16* recv[kArMaxRanks];          // rank r's receive buffer [source][rpr][ld]
    uint32_t* flags[kArMaxRanks];              // rank r's flags: [2][grid][size]
    uint32_t* counter;                         // local [grid]
    const __nv_bfloat16* residual; int ld_res; // local, all rows (null: none)
    __nv_bfloat16* out[kArMaxRanks]; int ldo;  // every rank's output buffer (peer pointers)
    uint32_t* status;
};

__global__ void __launch_bounds__(256) reduce_gather_kernel(const RgArgs a, const long long budget) {
    __shared__ bool s_fail;
    __shared__ uint32_t s_val;
    if (threadIdx.x == 0) { s_fail = false; s_val = a.counter[blockIdx.x] + 1u; }
    __syncthreads();
    const uint32_t val = s_val;
    const int per_row = a.n >> 3;
    if (a.partial != nullptr) {
        // CTA c pushes, for every owner, exactly the chunks that CTA c of that owner will reduce: barrier A below (same
        // CTA index on every rank) then covers them
        for (int p = 0; p < a.size; ++p) {
            const int o = (a.rank + p) % a.size;
            const int o0 = o * a.rpr, o1 = min(a.rows, o0 + a.rpr);
            const long long n_o = (long long)max(0, o1 - o0) * per_row;
            for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_o; c += (long long)gridDim.x * blockDim.x) {
                const int lr = (int)(c / per_row), col = (int)(c % per_row) << 3;
                const uint4 v = *reinterpret_cast<const uint4*>(a.partial + (size_t)(o0 + lr) * a.ld_partial + col);
                *reinterpret_cast<uint4*>(a.recv[o] + ((size_t)a.rank * a.rpr + lr) * a.ld + col) = v;
            }
        }
    }
    if (!peer_barrier(a.flags, a.size, a.rank, 0, val, &s_fail, budget)) {
        if (threadIdx.x == 0) set_status(a.status, PS_DEV_WAIT_TIMEOUT);
        return;
    }
    const int m0 = a.rank * a.rpr, m1 = min(a.rows, m0 + a.rpr);
    const long long chunks = (long long)max(0, m1 - m0) * per_row;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (long long)gridDim.x * blockDim.x) {
        const int lr = (int)(c / per_row), col = (int)(c % per_row) << 3;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const int row = m0 + lr;
        uint4 pv[kArMaxRanks];
#pragma unroll
        for (int r = 0; r < kArMaxRanks; ++r)            // all loads in flight before the first add
            if (r < a.size) pv[r] = __ldcv(reinterpret_cast<const uint4*>(a.src[r] + (size_t)(row - a.src_row0) * a.ld + col));
#pragma unroll
        for (int r = 0; r < kArMaxRanks; ++r)
            if (r < a.size) acc_bf16x8(acc, pv[r]);
        if (a.residual != nullptr) {
            const uint4 rv = *reinterpret_cast<const uint4*>(a.residual + (size_t)row * a.ld_res + col);
            const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = bf16x2_bits_to_f32x2(w[i]);
                acc[2 * i] = bf16_to_f32(f32_to_bf16(acc[2 * i])) + f.x;
                acc[2 * i + 1] = bf16_to_f32(f32_to_bf16(acc[2 * i + 1])) + f.y;
            }
        }
        const uint4 o = make_uint4(f32x2_to_bf16x2_bits(acc[0], acc[1]), f32x2_to_bf16x2_bits(acc[2], acc[3]),
                                   f32x2_to_bf16x2_bits(acc[4], acc[5]), f32x2_to_bf16x2_bits(acc[6], acc[7]));
        for (int p = 0; p < a.size; ++p) {
            const int pr = (a.rank + p) % a.size;          // start with myself, spread the peers over the links
            *reinterpret_cast<uint4*>(a.out[pr] + (size_t)row * a.ldo + col) = o;
        }
    }
    if (!peer_barrier(a.flags, a.size, a.rank, 1, val, &s_fail, budget)) {
        if (threadIdx.x == 0) set_status(a.status, PS_DEV_WAIT_TIMEOUT);
        return;
    }
    if (threadIdx.x == 0) a.counter[blockIdx.x] = val;
}

}  // namespace ps

// `args` points to a host copy of ps::RgArgs.  n and the row pitches must be multiples of 8; `grid` the same on every rank.
PS_API int ps_tp_reduce_gather(const void* args, int grid, cudaStream_t stream) {
    using namespace ps;
    const RgArgs& a = *reinterpret_cast<const RgArgs*>(args);
    if (a.size < 1 || a.size > kArMaxRanks || a.rows <= 0 || (a.n & 7) || (a.ld & 7) || (a.ldo & 7) || (a.ld_res & 7) || grid < 1 ||
        a.rpr < 1 || (long long)a.rpr * a.size < a.rows)
        return (int)cudaErrorInvalidValue;
    reduce_gather_kernel<<<grid, 256, 0, stream>>>(a, g_ps_wait_budget_cycles);
    return PS_LAUNCH_CHECK();
}

// `args` points to a host copy of ps::ArArgs.  n must be a multiple of 8; all buffers 16-byte aligned.
// `grid` must be the same on every rank (flags are indexed by CTA).
PS_API int ps_allreduce(const void* args, int use_multimem, int grid, cudaStream_t stream) {
    using namespace ps;
    const ArArgs& a = *reinterpret_cast<const ArArgs*>(args);
    if (a.size < 1 || a.size > kArMaxRanks || a.rows <= 0 || (a.n & 7) || grid < 1) return (int)cudaErrorInvalidValue;
    if (use_multimem) {
        if (a.mc_in == nullptr || a.mc_res == nullptr || a.res_local == nullptr) return (int)cudaErrorInvalidValue;
        allreduce_multimem_kernel<<<grid, 256, 0, stream>>>(a, g_ps_wait_budget_cycles);
    } else {
        allreduce_peer_kernel<<<grid, 256, 0, stream>>>(a, g_ps_wait_budget_cycles);
    }
    return PS_LAUNCH_CHECK();
}
