// Streaming small-M linear (decode / verify hot path): weights flow HBM -> shared memory through the
// TMA engine, one contiguous bulk copy per (quad, k-step) unit.
//
// One persistent CTA per SM (16 warps).  Every warp owns a private ring of shared-memory slots and
// keeps it full with `cp.async.bulk` copies that complete on an mbarrier, so ~150 KB of weight bytes
// per SM are in flight with no register cost -- what 6.5 TB/s of HBM3e needs (bandwidth x loaded
// latency is ~10 MB across the chip).  The CTA's quads are processed in waves of 16; inside a wave the
// (quad, k-step) units are cut into 16 contiguous slices (one per warp), so every warp streams the same
// number of bytes whatever N and K are, and a warp's units are one sequential byte range in memory.
// Partial sums of a quad meet in shared memory and are combined in warp order.
//
// Prologue / epilogue fusion and the batch-invariance contract are described in gemv_core.cuh.
#include "gemv_core.cuh"
#include "ps_tcgen05.cuh"

namespace ps {

constexpr int kStThreads = 512;
constexpr int kStWarps = kStThreads / 32;
constexpr int kStWaveQuads = 16;   // fixed: the unit -> warp assignment must not depend on M
constexpr int kStMaxSlots = 4;     // ring depth per warp (the launcher may pick fewer to fit shared memory)

template <int WF> __host__ __device__ constexpr int slot_stride() { return (WTraits<WF>::kBlockBytes + 127) / 128 * 128; }

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(tc::smem_u32(bar)) : "memory");
}

// AMAX: greedy sampling fused into the epilogue (ps_linear_stream_argmax); a template parameter, so that the kernel every
// other projection uses is compiled without a trace of it
template <int WF, int MT, bool AMAX = false>
__global__ void __launch_bounds__(kStThreads, 1) linear_stream_kernel(const LinearSmallArgs a, uint32_t* status,
                                                                       const int n_slots, const long long budget) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using XS = typename WTraits<WF>::XS;
    using RD = RowDot<WF>;
    constexpr int CH = WTraits<WF>::kChunk;
    constexpr int R = kQuadRows;
    constexpr int kBlock = WTraits<WF>::kBlockBytes;
    constexpr int kSlot = slot_stride<WF>();
    const int kpad = gemv_kpad<WF>(a.K);
    // layout: [rings: warps x slots x slot stride][xs: MT x kpad][partial: wave quads x warps x R x MT]
    XS* xs = reinterpret_cast<XS*>(smem_raw + (size_t)kStWarps * n_slots * kSlot);
    float* partial = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + (size_t)kpad * MT * sizeof(XS));
    __shared__ __align__(8) uint64_t s_bar[kStWarps][kStMaxSlots];
    __shared__ float s_xscale_inv[MT], s_red[64];

    // Programmatic dependent launch: the next kernel in the stream may start (and prefetch its own
    // weights) while this one runs; it blocks in cudaGridDependencySynchronize() until this grid is done.
    cudaTriggerProgrammaticLaunchCompletion();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_quads = (a.N + R - 1) / R;
    const int steps = gemv_steps<WF>(a.K);
    constexpr int wave_first = kStWaveQuads;
    int quad_begin, quad_end;
    cta_range(n_quads, gridDim.x, blockIdx.x, quad_begin, quad_end);

    if (lane == 0) {
        for (int s = 0; s < n_slots; ++s) tc::mbar_init(&s_bar[warp][s], 1);
        tc::fence_barrier_init();
    }
    __syncwarp();
    unsigned char* my_ring = smem_raw + (size_t)warp * n_slots * kSlot;

    // ---- producer side (lane 0 of each warp): first ring fill happens before the activations exist
    QuadWalker L;
    L.init(quad_begin, quad_end, steps, warp, kStWarps, kStWaveQuads);
    int issued = 0;
    if (lane == 0) {
        for (int s = 0; s < n_slots && L.valid(); ++s) {
            tc::mbar_expect_tx(&s_bar[warp][s], kBlock);
            bulk_g2s(my_ring + (size_t)s * kSlot, a.w + ((size_t)L.q * steps + L.st) * kBlock, kBlock, &s_bar[warp][s]);
            L.next();
            ++issued;
        }
    }

    for (int i = threadIdx.x; i < kStWaveQuads * kStWarps * R * MT; i += kStThreads) partial[i] = 0.f;
    StageW sw;
    stage_load_norm_w<kStThreads>(a, sw);
    cudaGridDependencySynchronize();
    // the first wave's residual rows are needed only in the epilogue: pull them towards the SM now
    if (a.epilogue == EPI_RESIDUAL && a.residual != nullptr) {
        const int wq0 = min(wave_first, quad_end - quad_begin);
        for (int i = threadIdx.x; i < wq0 * MT; i += kStThreads) {
            const int ql = i / MT, m = i % MT;
            if (m < a.M) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.residual + (size_t)m * a.ld_res + (size_t)(quad_begin + ql) * R));
        }
    }
    stage_rows<WF, MT, kStThreads>(a, xs, kpad, s_xscale_inv, s_red, sw);
    __syncthreads();

    int consumed = 0;
    bool timed_out = false;
    [[maybe_unused]] unsigned long long amax_mine = 0ull;      // AMAX: this thread's best key (its batch row is threadIdx.x % MT)
    [[maybe_unused]] bool amax_bad = false;
    for (int wave_q0 = quad_begin; wave_q0 < quad_end; wave_q0 += kStWaveQuads) {
        const int wave_quads = min(kStWaveQuads, quad_end - wave_q0);
        const int total = wave_quads * steps;
        const int u0 = (total * warp) / kStWarps, u_end = (total * (warp + 1)) / kStWarps;
        float acc[R][MT];
        int cur_q = wave_q0 + u0 / steps, st = u0 % steps;
        bool dirty = false;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
        auto flush = [&]() {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float v = warp_sum(acc[r][m]);
                    if (lane == 0) partial[((cur_q - wave_q0) * kStWarps + warp) * (R * MT) + r * MT + m] = v;
                    acc[r][m] = 0.f;
                }
        };
        for (int u = u0; u < u_end; ++u) {
            const int slot = consumed % n_slots;
            // warp-uniform outcome: either every lane saw the copy land or the whole warp gives up
            if (!__all_sync(0xffffffffu, tc::mbar_wait(&s_bar[warp][slot], (uint32_t)(consumed / n_slots) & 1u, budget))) { timed_out = true; break; }
            const unsigned char* blk = my_ring + (size_t)slot * kSlot;
            const int k = st * 32 * CH + lane * (16 / (int)sizeof(XS));      // lane's first 16-byte group of the step
            uint4 w[R]; uint32_t sb[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                w[r] = *reinterpret_cast<const uint4*>(blk + r * 512 + lane * 16);
                sb[r] = RD::load_scale(blk, r, lane);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                uint32_t xm[RD::kXWords];
                RD::load_x(xs + (size_t)m * kpad + k, xm);
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r][m] = RD::dot(w[r], sb[r], xm, acc[r][m]);
            }
            dirty = true;
            ++consumed;
            __syncwarp();     // every lane is done reading the slot before it is refilled
            if (lane == 0 && L.valid()) {
                tc::mbar_expect_tx(&s_bar[warp][slot], kBlock);
                bulk_g2s(my_ring + (size_t)slot * kSlot, a.w + ((size_t)L.q * steps + L.st) * kBlock, kBlock, &s_bar[warp][slot]);
                L.next();
                ++issued;
            }
            if (++st == steps) { flush(); dirty = false; st = 0; ++cur_q; }
        }
        if (dirty) flush();
        __syncthreads();
        // ---- combine the warps' partial sums in warp order, apply the epilogue
        if (a.tp.size <= 1) {
            for (int i = threadIdx.x; i < wave_quads * MT; i += kStThreads) {
                const int ql = i / MT, m = i % MT;
                float v[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float s = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < kStWarps; ++w2) {
                        float* pp = &partial[(ql * kStWarps + w2) * (R * MT) + r * MT + m];
                        s += *pp;
                        *pp = 0.f;
                    }
                    v[r] = s * (a.w_gscale * s_xscale_inv[m]);
                }
                if (m < a.M) {
                    if constexpr (AMAX) {
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const int n = (wave_q0 + ql) * R + r;
                            if (n < a.N) {
                                if (!(fabsf(v[r]) <= 3.0e38f)) amax_bad = true;
                                const unsigned long long key = amax_key(v[r], n);
                                if (key > amax_mine) amax_mine = key;
                            }
                        }
                    }
                    if (!AMAX || a.out != nullptr) quad_epilogue(a, (wave_q0 + ql) * R, m, v);
                }
            }
        } else {
            // ---- tensor-parallel combine (see TpCombine)
            const TpCombine& tp = a.tp;
            __shared__ uint32_t s_val;
            if (threadIdx.x == 0) s_val = tp.counter[blockIdx.x] + 1u;
            __syncthreads();
            const uint32_t val = s_val;
            const size_t par_off = (size_t)(val & 1u) * tp.size * tp.max_rows * tp.n_pad;
            // 1. push this CTA's partial rows into every rank's receive buffer (slot = my rank)
            for (int i = threadIdx.x; i < wave_quads * MT; i += kStThreads) {
                const int ql = i / MT, m = i % MT;
                float v[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float s = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < kStWarps; ++w2) {
                        float* pp = &partial[(ql * kStWarps + w2) * (R * MT) + r * MT + m];
                        s += *pp;
                        *pp = 0.f;
                    }
                    v[r] = s * (a.w_gscale * s_xscale_inv[m]);
                }
                if (m < a.M) {
                    const size_t off = par_off + ((size_t)tp.rank * tp.max_rows + m) * tp.n_pad + (size_t)(wave_q0 + ql) * R;
                    const float4 pk = make_float4(v[0], v[1], v[2], v[3]);
                    for (int pr = 0; pr < tp.size; ++pr) *reinterpret_cast<float4*>(tp.recv[pr] + off) = pk;
                }
            }
            __syncthreads();
            // 2. publish: one system-scope release per peer, then 3. wait for the same CTA of every peer
            if (threadIdx.x < tp.size) {
                // the barrier above ordered the CTA's peer stores before this thread; the system-scope release
                // on the flag is cumulative over them, so no separate fence is needed
                uint32_t* f = tp.flags[threadIdx.x] + (size_t)blockIdx.x * tp.size + tp.rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(val) : "memory");
                const uint32_t* mine = tp.flags[tp.rank] + (size_t)blockIdx.x * tp.size + threadIdx.x;
                const long long t0 = clock64();
                uint32_t seen;
                do {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
                    if ((int32_t)(seen - val) >= 0) break;
                    if (clock64() - t0 > budget) { timed_out = true; break; }
                } while (true);
            }
            __syncthreads();
            if (threadIdx.x == 0) tp.counter[blockIdx.x] = val;
            // 4. add the partials in rank order (identical on every rank), then the residual epilogue
            const float* rbuf = tp.recv[tp.rank] + par_off;
            for (int i = threadIdx.x; i < wave_quads * MT; i += kStThreads) {
                const int ql = i / MT, m = i % MT;
                if (m >= a.M) continue;
                const int n0 = (wave_q0 + ql) * R;
                float v[R] = {0.f, 0.f, 0.f, 0.f};
                for (int pr = 0; pr < tp.size; ++pr) {
                    const float4 pk = __ldcv(reinterpret_cast<const float4*>(rbuf + ((size_t)pr * tp.max_rows + m) * tp.n_pad + n0));
                    v[0] += pk.x; v[1] += pk.y; v[2] += pk.z; v[3] += pk.w;
                }
                quad_epilogue(a, n0, m, v);
            }
        }
        // whichever thread's wait ran out, the whole CTA leaves and every warp's lane 0 reports and drains
        if (__syncthreads_or(timed_out ? 1 : 0)) { timed_out = true; break; }
    }
    if constexpr (AMAX) {
        // fused greedy sampling: CTA-level maximum per batch row in shared memory, one global atomic per row and CTA, and
        // the last CTA to arrive publishes the winners and re-arms the state for the next launch (nobody waits)
        __shared__ unsigned long long s_amax[8];
        __shared__ int s_amax_last;
        if (threadIdx.x < 8) s_amax[threadIdx.x] = 0ull;
        __syncthreads();
        if (amax_mine != 0ull) atomicMax(&s_amax[threadIdx.x % MT], amax_mine);      // a thread only ever sees row threadIdx.x % MT
        const int any_bad = __syncthreads_or(amax_bad ? 1 : 0);
        if ((int)threadIdx.x < a.M && s_amax[threadIdx.x] != 0ull) atomicMax(&a.amax_best[threadIdx.x], s_amax[threadIdx.x]);
        if (threadIdx.x == 0 && any_bad) atomicOr(&a.amax_ctl[1], 1u);
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_amax_last = atomicAdd(&a.amax_ctl[0], 1u) == gridDim.x - 1 ? 1 : 0;
        __syncthreads();
        if (s_amax_last) {
            __threadfence();
            const unsigned int bad = *reinterpret_cast<volatile unsigned int*>(&a.amax_ctl[1]);
            if ((int)threadIdx.x < a.M) {
                const unsigned long long key = atomicMax(&a.amax_best[threadIdx.x], 0ull);
                a.amax_tokens[threadIdx.x] = (bad || key == 0ull) ? -1 : (int)(0xffffffffu - (uint32_t)(key & 0xffffffffull));
                a.amax_best[threadIdx.x] = 0ull;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                if (bad) set_status(status, PS_DEV_NONFINITE);
                a.amax_ctl[0] = 0u; a.amax_ctl[1] = 0u;
            }
        }
    }
    if (timed_out && lane == 0) {
        // A copy never completed.  Report it and give copies still in flight a bounded chance to land
        // before the CTA (and its shared memory) goes away.
        set_status(status, PS_DEV_WAIT_TIMEOUT);
        for (int c = consumed; c < issued; ++c) tc::mbar_wait(&s_bar[warp][c % n_slots], (uint32_t)(c / n_slots) & 1u, budget);
    }
}

static int g_st_sm_count = 0, g_st_pdl = 1;

template <int WF, int MT, bool AMAX = false>
static int launch_stream(const LinearSmallArgs& a, uint32_t* status, cudaStream_t stream) {
    const int kpad = gemv_kpad<WF>(a.K);
    const size_t fixed = (size_t)kpad * MT * sizeof(typename WTraits<WF>::XS) +
                         sizeof(float) * kStWaveQuads * kStWarps * kQuadRows * MT;
    const size_t budget = 224 * 1024;
    int slots = kStMaxSlots;
    while (slots >= 2 && fixed + (size_t)kStWarps * slots * slot_stride<WF>() > budget) --slots;
    if (slots < 2) return -1;      // activations do not fit next to a ring: the caller splits M
    const size_t smem = fixed + (size_t)kStWarps * slots * slot_stride<WF>();
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(linear_stream_kernel<WF, MT, AMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        attr_set = true;
    }
    const int n_quads = (a.N + kQuadRows - 1) / kQuadRows;
    const int grid = n_quads < g_st_sm_count ? n_quads : g_st_sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kStThreads); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_st_pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, linear_stream_kernel<WF, MT, AMAX>, a, status, slots, g_ps_wait_budget_cycles);
}

template <int WF>
static int stream_dispatch_m(const LinearSmallArgs& a, uint32_t* status, cudaStream_t stream) {
    if (a.M <= 1) return launch_stream<WF, 1>(a, status, stream);
    if (a.M <= 2) return launch_stream<WF, 2>(a, status, stream);
    if (a.M <= 4) return launch_stream<WF, 4>(a, status, stream);
    if (a.M <= 8) return launch_stream<WF, 8>(a, status, stream);
    return -1;
}

template <int WF>
static int stream_dispatch_m_amax(const LinearSmallArgs& a, uint32_t* status, cudaStream_t stream) {
    if (a.M <= 1) return launch_stream<WF, 1, true>(a, status, stream);
    if (a.M <= 2) return launch_stream<WF, 2, true>(a, status, stream);
    if (a.M <= 4) return launch_stream<WF, 4, true>(a, status, stream);
    if (a.M <= 8) return launch_stream<WF, 8, true>(a, status, stream);
    return -1;
}

static void stream_init_once() {
    if (g_st_sm_count != 0) return;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_st_sm_count, cudaDevAttrMultiProcessorCount, dev);
    const char* e = getenv("PS_PDL");
    g_st_pdl = (e == nullptr || e[0] != '0') ? 1 : 0;
}

}  // namespace ps

// y = epilogue( prologue(x) . W^T ) for M <= 8 over tiled weights.  Returns a cudaError_t value, or -1
// (nothing launched) when M rows of K activations do not fit in shared memory next to the ring.
PS_API int ps_linear_stream(int wfmt, const void* x, int M, int N, int K, int ldx, const void* w_tiled,
                            float w_gscale, int prologue, const void* norm_w, float eps, const void* gate,
                            int ld_gate, int epilogue, const void* residual, int ld_res, void* out, int ldo,
                            int out_f32, void* xn_out, const void* tp_combine, void* status, cudaStream_t stream) {
    using namespace ps;
    stream_init_once();
    if (M < 1 || M > 8 || (K % 32) != 0 || (ldx % 8) != 0 || ((uintptr_t)w_tiled % 16) != 0)
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && (N & 1)) return (int)cudaErrorInvalidValue;
    LinearSmallArgs a;
    a.x = (const __nv_bfloat16*)x; a.M = M; a.N = N; a.K = K; a.ldx = ldx;
    a.w = (const uint8_t*)w_tiled; a.w_gscale = w_gscale;
    a.prologue = prologue; a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps;
    a.gate = (const __nv_bfloat16*)gate; a.ld_gate = ld_gate;
    a.epilogue = epilogue; a.residual = (const __nv_bfloat16*)residual; a.ld_res = ld_res;
    a.out = out; a.ldo = ldo; a.out_f32 = out_f32; a.xn_out = (__nv_bfloat16*)xn_out;
    a.amax_best = nullptr; a.amax_ctl = nullptr; a.amax_tokens = nullptr;
    if (tp_combine != nullptr) {
        a.tp = *reinterpret_cast<const TpCombine*>(tp_combine);
        if (a.tp.size > kTpMaxRanks || M > a.tp.max_rows || ((N + 3) / 4 * 4) > a.tp.n_pad || epilogue == EPI_SWIGLU)
            return (int)cudaErrorInvalidValue;
    } else {
        a.tp.size = 0;
    }
    switch (wfmt) {
        case W_BF16: return stream_dispatch_m<W_BF16>(a, (uint32_t*)status, stream);
        case W_NVFP4: return stream_dispatch_m<W_NVFP4>(a, (uint32_t*)status, stream);
        case W_MXFP8: return stream_dispatch_m<W_MXFP8>(a, (uint32_t*)status, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// The same projection with greedy sampling fused into it (the lm_head of a decode step): `tokens[m]` receives the index of
// row m's largest output (ties to the lower index, -1 and PS_DEV_NONFINITE if a value is not finite), in the same launch.
// `state` is 8 x uint64 + 2 x uint32 of device memory, zeroed once by the caller and kept zero between launches by the
// kernel.  `out` may be null: the logits are then never written.  No tensor-parallel combine, store epilogue only.
// Reference: src/phaseshift/models/qwen35/kernels/optimized/sampling.hip:114-204 (arg-max contract).
PS_API int ps_linear_stream_argmax(int wfmt, const void* x, int M, int N, int K, int ldx, const void* w_tiled, float w_gscale,
                                   int prologue, const void* norm_w, float eps, void* out, int ldo, void* state, void* tokens,
                                   void* status, cudaStream_t stream) {
    using namespace ps;
    stream_init_once();
    if (M < 1 || M > 8 || (K % 32) != 0 || (ldx % 8) != 0 || ((uintptr_t)w_tiled % 16) != 0 || state == nullptr || tokens == nullptr)
        return (int)cudaErrorInvalidValue;
    LinearSmallArgs a;
    a.x = (const __nv_bfloat16*)x; a.M = M; a.N = N; a.K = K; a.ldx = ldx;
    a.w = (const uint8_t*)w_tiled; a.w_gscale = w_gscale;
    a.prologue = prologue; a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps;
    a.gate = nullptr; a.ld_gate = 0; a.epilogue = EPI_STORE; a.residual = nullptr; a.ld_res = 0;
    a.out = out; a.ldo = ldo; a.out_f32 = 1; a.xn_out = nullptr; a.tp.size = 0;
    a.amax_best = (unsigned long long*)state; a.amax_ctl = (unsigned int*)((unsigned long long*)state + 8); a.amax_tokens = (int*)tokens;
    switch (wfmt) {
        case W_BF16: return stream_dispatch_m_amax<W_BF16>(a, (uint32_t*)status, stream);
        case W_NVFP4: return stream_dispatch_m_amax<W_NVFP4>(a, (uint32_t*)status, stream);
        case W_MXFP8: return stream_dispatch_m_amax<W_MXFP8>(a, (uint32_t*)status, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// Largest M the streaming kernel can stage for a format and K (0 if even one row does not fit).
PS_API int ps_linear_stream_max_rows(int wfmt, int K) {
    using namespace ps;
    for (int mt = 8; mt >= 1; mt >>= 1) {
        size_t per, slot;
        if (wfmt == W_BF16) { per = (size_t)gemv_kpad<W_BF16>(K) * 4; slot = slot_stride<W_BF16>(); }
        else if (wfmt == W_NVFP4) { per = (size_t)gemv_kpad<W_NVFP4>(K) * 2; slot = slot_stride<W_NVFP4>(); }
        else { per = (size_t)gemv_kpad<W_MXFP8>(K) * 2; slot = slot_stride<W_MXFP8>(); }
        const size_t fixed = per * mt + sizeof(float) * kStWaveQuads * kStWarps * kQuadRows * mt;
        if (fixed + (size_t)kStWarps * 2 * slot <= 224 * 1024) return mt;
    }
    return 0;
}
