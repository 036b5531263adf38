// Gated DeltaNet, chunked (prefill) form: four launches per layer.
//
// With G_t the running sum of the log decays g inside a 64-row chunk, D_t = exp(G_t) and S0 the state
// entering the chunk, the exact recurrence
//     S <- d_t S ;  delta_t = beta_t (v_t - S^T k_t) ;  S <- S + k_t delta_t^T ;  o_t = S^T q_t
// is equivalent to
//     (I + A) Delta = B,  A_ts = beta_t (D_t/D_s)(k_t.k_s) for s < t,  B_t = beta_t (v_t - D_t S0^T k_t)
//     o_t = D_t S0^T q_t + sum_{s<=t} (D_t/D_s)(q_t.k_s) delta_s ,   S_C = D_C S0 + sum_s (D_C/D_s) k_s delta_s^T
// and, with T = (I + A)^-1 (unit lower triangular, independent of the state),
//     Delta = U - W S0 ,   U = T diag(beta) V ,   W = T diag(beta D) K .
// Everything that does not depend on S0 is computed for all chunks at once:
//
//   1. gdn_chunk_prep : one CTA per (chunk, value head): causal depthwise conv (kernel 4) + SiLU with the
//      taps sliding through registers, L2 normalisation (q also scaled by Dk^-0.5), beta = sigmoid(b),
//      g = -exp(A_log) softplus(a + dt_bias); then A and QKd from K K^T and Q K^T on the tensor cores, T by
//      forward substitution on the identity (one thread per column, out of registers), W and U as
//      tensor-core products with T, and the decayed operands Qd = D q, Kd = (D_C/D_s) k, written to scratch.
//   2. gdn_history : stores the raw inputs of each sequence's last rows in the conv ring (a separate
//      launch so no CTA reads history that another CTA of the same step is overwriting).
//   3. gdn_chunk_scan_tc : one CTA per (sequence, value head, 64-column slice of Dv) walks the chunks:
//      Delta = U - W S0 ;  O = Qd S0 + QKd Delta ;  S = D_C S0 + Kd^T Delta.  Three small tensor-core
//      products per chunk, no serial solve on the critical path; the state stays in accumulator registers.
//      (gdn_chunk_scan is the same walk with fp32 CUDA-core products, selected by PS_GDN_SCAN=fp32.)
//   4. gdn_post : RMSNorm over the head's Dv outputs (direct weight) * SiLU(z) -> bf16.
//
// All decay ratios have s <= t and g <= 0, so every exponential is <= 1.  The state and every accumulation
// are fp32; the tensor-core products take TF32 operands (mma.sync m16n8k8, round-to-nearest copies).
// The reference's chunked kernel (src/phaseshift/models/qwen35/kernels/optimized/gdn/recurrence.hip:
// 128-519) uses chunk 32, bf16 WMMA products (hi+lo split in "exact" mode) and a 32-step serial forward
// substitution per column inside the sequential walk.  Decode and speculative verification keep using
// the row-sequential kernel (gdn_recurrent.cu), whose per-row arithmetic is independent of the batch.
#include "ps_common.cuh"

namespace ps {

struct GdnSeqDesc2 { int row_start; int n_rows; int slot; int pos_start; };

constexpr int kChunk = 64;
constexpr int kSlice = 64;     // Dv columns per scan CTA
constexpr int kTP = 68;        // pitch of T rows (floats), multiple of 4 for 16-byte broadcast loads

struct GdnPrepArgs {
    const __nv_bfloat16* proj; int ld_proj;      // [rows, ld]: [q | k | v | z | b | a]
    int Hk, Hv, Dk, Dv;
    const __nv_bfloat16* conv_w; const float* A_log; const float* dt_bias;
    __nv_bfloat16* conv_state; int ring;
    const int* row_slot; const int* row_pos;
    const GdnSeqDesc2* seqs; int n_seqs;
    int min_rows;                                // sequences with at most this many rows are left to the row kernel
    float* scratch;                              // per (chunk, head): W, Qd, Kd [64,Dk]; U [64,Dv]; QKd [64,64]
    float* dc;                                   // per (chunk, head): D_C
    int round_tf32;                              // 1: W, Qd, Kd, QKd are stored rounded to TF32 (the tensor-core scan copies them
                                                 // into shared memory asynchronously and cannot round on the way)
};

__host__ __device__ inline size_t chunk_scratch_floats(int Dk, int Dv) { return (size_t)kChunk * (3 * Dk + Dv + kChunk); }

// Locate global chunk `gc` (chunks are numbered sequence by sequence): returns false when out of range.
__device__ __forceinline__ bool find_chunk(const GdnSeqDesc2* seqs, int n_seqs, int min_rows, int gc, GdnSeqDesc2& sd, int& chunk) {
    int base = 0;
    for (int s = 0; s < n_seqs; ++s) {
        const GdnSeqDesc2 d = seqs[s];
        const int nc = d.n_rows > min_rows && d.slot >= 0 ? (d.n_rows + kChunk - 1) / kChunk : 0;
        if (gc < base + nc) { sd = d; chunk = gc - base; return true; }
        base += nc;
    }
    return false;
}

// TF32 tensor-core helpers (operands rounded to nearest TF32, fp32 accumulation)
__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const float (&a)[4], float b0, float b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])), "r"(__float_as_uint(a[3])),
                   "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// grid = (max chunks, Hv), block = 256 threads, two CTAs per SM (shared memory: Q and K tiles, the raw q|k input tile
// that A, T and the block-row temporaries later overwrite; V is convolved straight from global memory into Q's tile
// once Q is dead).
template <int DK, int DV>
__global__ void __launch_bounds__(256, 2) gdn_chunk_prep_kernel(const GdnPrepArgs a) {
    static_assert(DV <= DK && 256 % DK == 0 && 512 % DV == 0, "tile aliasing and the conv partition assume these");
    constexpr int CH = 2 * DK + DV, CQK = 2 * DK, PK = DK + 4, PV = DV + 4, RAWR = kChunk + 3;
    extern __shared__ __align__(16) float sm[];
    float* sQ = sm;                        // [64][DK+4]; after the decayed operands are written: V [64][DV+4]
    float* sK = sQ + kChunk * PK;          // [64][DK+4]
    float* sV = sQ;
    float* sG = sK + kChunk * PK;          // [64]
    float* sBeta = sG + kChunk;            // [64]
    float* sU = sBeta + kChunk;            // union: raw bf16 q|k tile [67][2 DK], later A [64][65], T [64][68], M [3][16][17]
    __nv_bfloat16* sRaw = reinterpret_cast<__nv_bfloat16*>(sU);
    float* sA = sU;
    float* sT = sA + kChunk * 65;          // 64 * 65 floats keep the T rows 16-byte aligned
    float* sM = sT + kChunk * kTP;

    GdnSeqDesc2 sd; int chunk;
    if (!find_chunk(a.seqs, a.n_seqs, a.min_rows, blockIdx.x, sd, chunk)) return;
    const int h = blockIdx.y, t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int r0 = chunk * kChunk, C = min(kChunk, sd.n_rows - r0);
    const size_t row0 = (size_t)sd.row_start + r0;
    const int pos0 = sd.pos_start + r0;
    const int hk = h / (a.Hv / a.Hk);
    const int q_off = hk * DK, k_off = a.Hk * DK + hk * DK, v_off = 2 * a.Hk * DK + h * DV;
    const int b_off = 2 * a.Hk * DK + 2 * a.Hv * DV + h, a_off = b_off + a.Hv;
    const __nv_bfloat16* hist = a.conv_state + ((size_t)sd.slot * a.Hv + h) * a.ring * CH;
    float* scr = a.scratch + ((size_t)blockIdx.x * a.Hv + h) * chunk_scratch_floats(DK, DV);
    float* gW = scr; float* gQd = gW + kChunk * DK; float* gKd = gQd + kChunk * DK;
    float* gU = gKd + kChunk * DK; float* gQK = gU + kChunk * DV;

    // ---- stage the raw inputs of rows -3 .. 63 (this head's q | k channels) with wide loads
    {
        const bool vec = (a.ld_proj % 8) == 0;
        constexpr int PPR = CQK / 8;
        for (int p = t; p < RAWR * PPR; p += 256) {
            const int rr = p / PPR - 3, c = (p % PPR) * 8;
            const int gc = c < DK ? q_off + c : k_off + (c - DK);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (rr < C && pos0 + rr >= 0) {
                if (r0 + rr >= 0) {
                    const __nv_bfloat16* src = a.proj + (size_t)((long long)row0 + rr) * a.ld_proj + gc;
                    if (vec) v = __ldg(reinterpret_cast<const uint4*>(src));
                    else {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) w[j] = (uint32_t)__bfloat16_as_ushort(src[2 * j]) | ((uint32_t)__bfloat16_as_ushort(src[2 * j + 1]) << 16);
                        v = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
                    v = *reinterpret_cast<const uint4*>(hist + (size_t)((pos0 + rr) % a.ring) * CH + c);
                }
            }
            *reinterpret_cast<uint4*>(sRaw + (rr + 3) * CQK + c) = v;
        }
    }
    // ---- beta and the running log decay (last warp, two 32-wide halves)
    if (warp == 7) {
        float g0 = 0.f, g1 = 0.f, b0 = 0.f, b1 = 0.f;
        const float Aexp = -__expf(a.A_log[h]), dtb = a.dt_bias[h];
        if (lane < C) {
            const __nv_bfloat16* pr = a.proj + (row0 + lane) * a.ld_proj;
            b0 = sigmoid_f(bf16_to_f32(pr[b_off])); g0 = Aexp * softplus_f(bf16_to_f32(pr[a_off]) + dtb);
        }
        if (lane + 32 < C) {
            const __nv_bfloat16* pr = a.proj + (row0 + lane + 32) * a.ld_proj;
            b1 = sigmoid_f(bf16_to_f32(pr[b_off])); g1 = Aexp * softplus_f(bf16_to_f32(pr[a_off]) + dtb);
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n0 = __shfl_up_sync(0xffffffffu, g0, o), n1 = __shfl_up_sync(0xffffffffu, g1, o);
            if (lane >= o) { g0 += n0; g1 += n1; }
        }
        const float tot0 = __shfl_sync(0xffffffffu, g0, 31);
        sG[lane] = g0; sG[lane + 32] = g1 + tot0;
        sBeta[lane] = b0; sBeta[lane + 32] = b1;
    }
    __syncthreads();
    // ---- conv + SiLU of q and k: a thread owns a channel pair over a run of rows and slides its taps through registers
    {
        constexpr int PARTS = 256 / DK, RUN = kChunk / PARTS;           // DK channel pairs x PARTS row runs = 256 threads
        const int c = 2 * (t % DK), rb = (t / DK) * RUN;
        const int gc = c < DK ? q_off + c : k_off + (c - DK);
        const uint4 wraw = *reinterpret_cast<const uint4*>(a.conv_w + (size_t)gc * 4);     // two channels x four taps
        const float2 wa01 = bf16x2_bits_to_f32x2(wraw.x), wa23 = bf16x2_bits_to_f32x2(wraw.y);
        const float2 wb01 = bf16x2_bits_to_f32x2(wraw.z), wb23 = bf16x2_bits_to_f32x2(wraw.w);
        const uint32_t* col = reinterpret_cast<const uint32_t*>(sRaw + c) + rb * (CQK / 2);
        float2 x3 = bf16x2_bits_to_f32x2(col[0 * (CQK / 2)]), x2 = bf16x2_bits_to_f32x2(col[1 * (CQK / 2)]);
        float2 x1 = bf16x2_bits_to_f32x2(col[2 * (CQK / 2)]);
        float* dst = (c < DK ? sQ + c : sK + (c - DK)) + rb * PK;
#pragma unroll 8
        for (int r = 0; r < RUN; ++r) {
            const float2 x0 = bf16x2_bits_to_f32x2(col[(r + 3) * (CQK / 2)]);
            float ya = wa01.x * x3.x; ya = fmaf(wa01.y, x2.x, ya); ya = fmaf(wa23.x, x1.x, ya); ya = fmaf(wa23.y, x0.x, ya);
            float yb = wb01.x * x3.y; yb = fmaf(wb01.y, x2.y, yb); yb = fmaf(wb23.x, x1.y, yb); yb = fmaf(wb23.y, x0.y, yb);
            x3 = x2; x2 = x1; x1 = x0;
            *reinterpret_cast<float2*>(dst + r * PK) = make_float2(silu_f(ya), silu_f(yb));
        }
    }
    __syncthreads();
    // ---- L2 norms: warp w owns rows 8w .. 8w+7
    for (int r = warp * 8; r < warp * 8 + 8; ++r) {
        float qq = 0.f, kk = 0.f;
        for (int d = lane; d < DK; d += 32) { const float qv = sQ[r * PK + d], kv = sK[r * PK + d]; qq += qv * qv; kk += kv * kv; }
        qq = warp_sum(qq); kk = warp_sum(kk);
        const float qn = rsqrtf(qq + 1e-6f) * rsqrtf((float)DK), kn = rsqrtf(kk + 1e-6f);
        for (int d = lane; d < DK; d += 32) { sQ[r * PK + d] *= qn; sK[r * PK + d] *= kn; }
    }
    __syncthreads();
    // ---- A (strictly lower) and QKd (lower incl. diagonal) on the tensor cores: warp -> rows 16 mt .., columns
    //      32 ch .. 32 ch + 31; K K^T and Q K^T share the B fragments (B[k = d][n = s] = K[s][d])
    {
        const int g = lane >> 2, tq = lane & 3, mt = warp & 3, ch = warp >> 2;
        float kk[4][4], qk[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) { kk[nt][0] = kk[nt][1] = kk[nt][2] = kk[nt][3] = 0.f; qk[nt][0] = qk[nt][1] = qk[nt][2] = qk[nt][3] = 0.f; }
        if (ch * 32 <= 16 * mt + 15) {                      // tiles entirely above the diagonal stay zero
            const float* kr = sK + (16 * mt + g) * PK + tq;
            const float* qr = sQ + (16 * mt + g) * PK + tq;
#pragma unroll 4
            for (int ks = 0; ks < DK / 8; ++ks) {
                const float ak[4] = {to_tf32(kr[8 * ks]), to_tf32(kr[8 * PK + 8 * ks]), to_tf32(kr[8 * ks + 4]), to_tf32(kr[8 * PK + 8 * ks + 4])};
                const float aq[4] = {to_tf32(qr[8 * ks]), to_tf32(qr[8 * PK + 8 * ks]), to_tf32(qr[8 * ks + 4]), to_tf32(qr[8 * PK + 8 * ks + 4])};
                const float* kb = sK + (32 * ch + g) * PK + 8 * ks + tq;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const float b0 = to_tf32(kb[8 * nt * PK]), b1 = to_tf32(kb[8 * nt * PK + 4]);
                    mma_tf32(kk[nt], ak, b0, b1);
                    mma_tf32(qk[nt], aq, b0, b1);
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int tt = 16 * mt + g + (e >> 1) * 8, ss = 32 * ch + 8 * nt + 2 * tq + (e & 1);
                const float dec = ss <= tt ? __expf(sG[tt] - sG[ss]) : 0.f;
                sA[tt * 65 + ss] = ss < tt ? sBeta[tt] * dec * kk[nt][e] : 0.f;
                gQK[tt * kChunk + ss] = a.round_tf32 ? to_tf32(dec * qk[nt][e]) : dec * qk[nt][e];
            }
    }
    __syncthreads();
    // ---- raw v inputs of this thread's conv run, requested now and used once Q's tile is free
    constexpr int VPARTS = 512 / DV, VRUN = kChunk / VPARTS;             // DV / 2 channel pairs x VPARTS row runs = 256 threads
    const int vc = 2 * (t % (DV / 2)), vrb = (t / (DV / 2)) * VRUN;
    uint32_t vraw[VRUN + 3];
    {
        const bool even = (a.ld_proj & 1) == 0;
#pragma unroll
        for (int i = 0; i < VRUN + 3; ++i) {
            const int rr = vrb + i - 3;
            uint32_t v = 0;
            if (rr < C && pos0 + rr >= 0) {
                if (r0 + rr >= 0) {
                    const __nv_bfloat16* src = a.proj + (size_t)((long long)row0 + rr) * a.ld_proj + v_off + vc;
                    v = even ? __ldg(reinterpret_cast<const uint32_t*>(src))
                             : ((uint32_t)__bfloat16_as_ushort(src[0]) | ((uint32_t)__bfloat16_as_ushort(src[1]) << 16));
                } else {
                    v = *reinterpret_cast<const uint32_t*>(hist + (size_t)((pos0 + rr) % a.ring) * CH + CQK + vc);
                }
            }
            vraw[i] = v;
        }
    }
    // ---- T = (I + A)^-1, diagonal 16x16 blocks: thread (block b, column j) solves by forward substitution out of
    //      registers; meanwhile the other warps write the decayed operands
    if (t < kChunk) {
        const int b = t >> 4, j = t & 15;
        const float* Ab = sA + (16 * b) * 65 + 16 * b;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float acc0 = i == j ? 1.f : 0.f, acc1 = 0.f;
#pragma unroll
            for (int k = 0; k < i; ++k) { if (k & 1) acc1 = fmaf(-Ab[i * 65 + k], x[k], acc1); else acc0 = fmaf(-Ab[i * 65 + k], x[k], acc0); }
            x[i] = acc0 + acc1;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) sT[(16 * b + i) * kTP + 16 * b + j] = x[i];
    } else {
        const float GC = sG[kChunk - 1];
        for (int i = t - kChunk; i < kChunk * DK / 4; i += 256 - kChunk) {
            const int r = (i * 4) / DK, d = (i * 4) % DK;
            const float eq = __expf(sG[r]), ek = __expf(GC - sG[r]);
            const float4 q = *reinterpret_cast<const float4*>(sQ + r * PK + d), k = *reinterpret_cast<const float4*>(sK + r * PK + d);
            float4 qd = make_float4(eq * q.x, eq * q.y, eq * q.z, eq * q.w), kd = make_float4(ek * k.x, ek * k.y, ek * k.z, ek * k.w);
            if (a.round_tf32) {
                qd = make_float4(to_tf32(qd.x), to_tf32(qd.y), to_tf32(qd.z), to_tf32(qd.w));
                kd = make_float4(to_tf32(kd.x), to_tf32(kd.y), to_tf32(kd.z), to_tf32(kd.w));
            }
            reinterpret_cast<float4*>(gQd)[i] = qd;
            reinterpret_cast<float4*>(gKd)[i] = kd;
        }
        if (t == kChunk) a.dc[(size_t)blockIdx.x * a.Hv + h] = __expf(GC);
    }
    __syncthreads();
    // ---- conv + SiLU of v into Q's tile (Q is dead: A, QKd and Qd are done)
    {
        const int gc = v_off + vc;
        const uint4 wraw = *reinterpret_cast<const uint4*>(a.conv_w + (size_t)gc * 4);
        const float2 wa01 = bf16x2_bits_to_f32x2(wraw.x), wa23 = bf16x2_bits_to_f32x2(wraw.y);
        const float2 wb01 = bf16x2_bits_to_f32x2(wraw.z), wb23 = bf16x2_bits_to_f32x2(wraw.w);
        float2 x3 = bf16x2_bits_to_f32x2(vraw[0]), x2 = bf16x2_bits_to_f32x2(vraw[1]), x1 = bf16x2_bits_to_f32x2(vraw[2]);
        float* dst = sV + vrb * PV + vc;
#pragma unroll
        for (int r = 0; r < VRUN; ++r) {
            const float2 x0 = bf16x2_bits_to_f32x2(vraw[r + 3]);
            float ya = wa01.x * x3.x; ya = fmaf(wa01.y, x2.x, ya); ya = fmaf(wa23.x, x1.x, ya); ya = fmaf(wa23.y, x0.x, ya);
            float yb = wb01.x * x3.y; yb = fmaf(wb01.y, x2.y, yb); yb = fmaf(wb23.x, x1.y, yb); yb = fmaf(wb23.y, x0.y, yb);
            x3 = x2; x2 = x1; x1 = x0;
            *reinterpret_cast<float2*>(dst + r * PV) = make_float2(silu_f(ya), silu_f(yb));
        }
    }
    // ---- T, block rows 1 .. 3: T_ij = -T_ii (sum_{k = j .. i-1} A_ik T_kj) for all j < i at once
    for (int bi = 1; bi < 4; ++bi) {
        for (int e = t; e < bi * 256; e += 256) {
            const int bj = e >> 8, r = (e >> 4) & 15, c = e & 15;
            const float* Ar = sA + (16 * bi + r) * 65;
            float acc0 = 0.f, acc1 = 0.f;
            for (int k = 16 * bj; k < 16 * bi; k += 2) {
                acc0 = fmaf(Ar[k], sT[k * kTP + 16 * bj + c], acc0);
                acc1 = fmaf(Ar[k + 1], sT[(k + 1) * kTP + 16 * bj + c], acc1);
            }
            sM[(bj * 16 + r) * 17 + c] = acc0 + acc1;
        }
        __syncthreads();
        for (int e = t; e < bi * 256; e += 256) {
            const int bj = e >> 8, r = (e >> 4) & 15, c = e & 15;
            const float* Tr = sT + (16 * bi + r) * kTP + 16 * bi;
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < 16; ++k) acc = fmaf(Tr[k], sM[(bj * 16 + k) * 17 + c], acc);     // T_ii is zero above its diagonal
            sT[(16 * bi + r) * kTP + 16 * bj + c] = -acc;
        }
        __syncthreads();
    }
    // ---- W = T diag(beta D) K (warps 0-3) and U = T diag(beta) V (warps 4-7) on the tensor cores: warp -> rows
    //      16 mt .., all columns of its matrix; T is lower triangular, so k-steps beyond the row tile are skipped
    {
        const int g = lane >> 2, tq = lane & 3, mt = warp & 3;
        const bool isW = warp < 4;
        constexpr int NTW = (DK > DV ? DK : DV) / 8;
        const int ntiles = (isW ? DK : DV) / 8;
        const float* src = isW ? sK : sV;
        const int pitch = isW ? PK : PV;
        float acc[NTW][4];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
        const float* tr = sT + (16 * mt + g) * kTP + tq;
        for (int ks = 0; ks < 2 * mt + 2; ++ks) {
            const float at[4] = {to_tf32(tr[8 * ks]), to_tf32(tr[8 * kTP + 8 * ks]), to_tf32(tr[8 * ks + 4]), to_tf32(tr[8 * kTP + 8 * ks + 4])};
            const int s0 = 8 * ks + tq, s1 = s0 + 4;
            const float f0 = sBeta[s0] * (isW ? __expf(sG[s0]) : 1.f), f1 = sBeta[s1] * (isW ? __expf(sG[s1]) : 1.f);
            const float* b0p = src + s0 * pitch + g;
            const float* b1p = src + s1 * pitch + g;
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt)
                if (nt < ntiles) mma_tf32(acc[nt], at, to_tf32(b0p[8 * nt] * f0), to_tf32(b1p[8 * nt] * f1));
        }
        float* dst = isW ? gW : gU;
        const int dp = isW ? DK : DV;
        if (isW && a.round_tf32) {
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) { acc[nt][0] = to_tf32(acc[nt][0]); acc[nt][1] = to_tf32(acc[nt][1]); acc[nt][2] = to_tf32(acc[nt][2]); acc[nt][3] = to_tf32(acc[nt][3]); }
        }
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt)
            if (nt < ntiles) {
                *reinterpret_cast<float2*>(dst + (size_t)(16 * mt + g) * dp + 8 * nt + 2 * tq) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(dst + (size_t)(16 * mt + g + 8) * dp + 8 * nt + 2 * tq) = make_float2(acc[nt][2], acc[nt][3]);
            }
    }
}


// True when `row` belongs to a sequence this launch handles (more than min_rows rows in the step).
__device__ __forceinline__ bool row_is_chunked(const GdnSeqDesc2* seqs, int n_seqs, int min_rows, int row) {
    for (int s = 0; s < n_seqs; ++s) {
        const GdnSeqDesc2 d = seqs[s];
        if (row >= d.row_start && row < d.row_start + d.n_rows) return d.n_rows > min_rows && d.slot >= 0;
    }
    return false;
}

// History for later steps: the raw inputs of each sequence's last `ring` rows.  Separate launch so the
// prepare CTAs of a step never race with history reads of earlier rows of the same step.
// grid = (Hv, ring, n_seqs): block (h, j, s) copies the j-th row from the end of sequence s.
__global__ void gdn_history_kernel(const GdnPrepArgs a) {
    const int h = blockIdx.x, j = blockIdx.y, t = threadIdx.x;
    const GdnSeqDesc2 sd = a.seqs[blockIdx.z];
    if (sd.slot < 0 || sd.n_rows <= a.min_rows || j >= sd.n_rows) return;
    const int r = sd.n_rows - 1 - j, pos = sd.pos_start + r;
    const int Dk = a.Dk, Dv = a.Dv, CH = 2 * Dk + Dv;
    const int hk = h / (a.Hv / a.Hk);
    const int q_off = hk * Dk, k_off = a.Hk * Dk + hk * Dk, v_off = 2 * a.Hk * Dk + h * Dv;
    const __nv_bfloat16* pr = a.proj + (size_t)(sd.row_start + r) * a.ld_proj;
    __nv_bfloat16* hist = a.conv_state + ((size_t)sd.slot * a.Hv + h) * a.ring * CH;
    for (int c = t; c < CH; c += blockDim.x) {
        const int gc = c < Dk ? q_off + c : (c < 2 * Dk ? k_off + (c - Dk) : v_off + (c - 2 * Dk));
        hist[(size_t)(pos % a.ring) * CH + c] = pr[gc];
    }
}

struct GdnScanArgs {
    const float* scratch; const float* dc;
    int Hv, Dv, n_seqs, min_rows;
    float* state;                 // [slots, Hv, Dk, Dv] fp32, updated in place
    const GdnSeqDesc2* seqs;
    float* o;                     // [rows, Hv, Dv] fp32
};

__device__ __forceinline__ void fma8(float (&acc)[8], float w, const float4& s0, const float4& s1) {
    acc[0] = fmaf(w, s0.x, acc[0]); acc[1] = fmaf(w, s0.y, acc[1]); acc[2] = fmaf(w, s0.z, acc[2]); acc[3] = fmaf(w, s0.w, acc[3]);
    acc[4] = fmaf(w, s1.x, acc[4]); acc[5] = fmaf(w, s1.y, acc[5]); acc[6] = fmaf(w, s1.z, acc[6]); acc[7] = fmaf(w, s1.w, acc[7]);
}

// grid = (Dv / kSlice, Hv, n_seqs), block = 256 threads.  Register tiles: 2 rows x 8 columns for the
// products with S0, 4 rows x 8 columns for the state update; all shared-memory operands are read as
// 16-byte vectors so the loops are bound by the FMA pipe, not by shared-memory bandwidth.
template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(const GdnScanArgs a) {
    constexpr int PK = DK + 4, PS = kSlice + 4;
    extern __shared__ __align__(16) float sm[];
    float* sW = sm;                          // [64][DK+4]
    float* sQd = sW + kChunk * PK;           // [64][DK+4]
    float* sKd = sQd + kChunk * PK;          // [64][DK+4]
    float* sS = sKd + kChunk * PK;           // [DK][kSlice+4]  state slice
    float* sD = sS + DK * PS;                // [64][kSlice+4]  U slice, then Delta
    float* sQK = sD + kChunk * PS;           // [64][65]

    const int slice = blockIdx.x, h = blockIdx.y, t = threadIdx.x, Hv = a.Hv, c0 = slice * kSlice;
    const GdnSeqDesc2 sd = a.seqs[blockIdx.z];
    if (sd.n_rows <= a.min_rows || sd.slot < 0) return;
    PS_CHECK(PS_SLOT_OK(sd.slot) && PS_ROWS_OK(sd.row_start, sd.n_rows));
    int gc = 0;
    for (int s = 0; s < (int)blockIdx.z; ++s) {
        const GdnSeqDesc2 d = a.seqs[s];
        if (d.n_rows > a.min_rows && d.slot >= 0) gc += (d.n_rows + kChunk - 1) / kChunk;
    }
    float* Sg = a.state + ((size_t)sd.slot * Hv + h) * DK * DV;
    for (int i = t; i < DK * kSlice / 4; i += 256) {
        const int d = (i * 4) / kSlice, c = (i * 4) % kSlice;
        *reinterpret_cast<float4*>(sS + d * PS + c) = *reinterpret_cast<const float4*>(Sg + (size_t)d * DV + c0 + c);
    }
    const int r2 = t / 8, cb = (t % 8) * 8;          // rows 2 r2, 2 r2 + 1 ; columns cb .. cb + 7

    for (int r0 = 0; r0 < sd.n_rows; r0 += kChunk, ++gc) {
        const int C = min(kChunk, sd.n_rows - r0);
        const size_t rowbase = (size_t)(sd.row_start + r0);
        const float* scr = a.scratch + ((size_t)gc * Hv + h) * chunk_scratch_floats(DK, DV);
        const float* gW = scr; const float* gQd = gW + kChunk * DK; const float* gKd = gQd + kChunk * DK;
        const float* gU = gKd + kChunk * DK; const float* gQK = gU + kChunk * DV;
        __syncthreads();
        for (int i = t; i < kChunk * DK / 4; i += 256) {
            const int r = (i * 4) / DK, d = (i * 4) % DK;
            *reinterpret_cast<float4*>(sW + r * PK + d) = __ldg(reinterpret_cast<const float4*>(gW) + i);
            *reinterpret_cast<float4*>(sQd + r * PK + d) = __ldg(reinterpret_cast<const float4*>(gQd) + i);
            *reinterpret_cast<float4*>(sKd + r * PK + d) = __ldg(reinterpret_cast<const float4*>(gKd) + i);
        }
        for (int i = t; i < kChunk * kChunk; i += 256) sQK[(i / kChunk) * 65 + (i % kChunk)] = __ldg(gQK + i);
        for (int i = t; i < kChunk * kSlice / 4; i += 256) {
            const int r = (i * 4) / kSlice, c = (i * 4) % kSlice;
            *reinterpret_cast<float4*>(sD + r * PS + c) = __ldg(reinterpret_cast<const float4*>(gU + (size_t)r * DV + c0 + c));
        }
        const float DC = a.dc[(size_t)gc * Hv + h];
        __syncthreads();
        // ---- Delta = U - W S0 and R = Qd S0
        float R0[8], R1[8];
        {
            float P0[8], P1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { P0[j] = P1[j] = R0[j] = R1[j] = 0.f; }
            const float* w0p = sW + (2 * r2) * PK; const float* q0p = sQd + (2 * r2) * PK;
#pragma unroll 2
            for (int d = 0; d < DK; d += 4) {
                const float4 w0 = *reinterpret_cast<const float4*>(w0p + d), w1 = *reinterpret_cast<const float4*>(w0p + PK + d);
                const float4 q0 = *reinterpret_cast<const float4*>(q0p + d), q1 = *reinterpret_cast<const float4*>(q0p + PK + d);
                const float wv0[4] = {w0.x, w0.y, w0.z, w0.w}, wv1[4] = {w1.x, w1.y, w1.z, w1.w};
                const float qv0[4] = {q0.x, q0.y, q0.z, q0.w}, qv1[4] = {q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                for (int dd = 0; dd < 4; ++dd) {
                    const float4 s0 = *reinterpret_cast<const float4*>(sS + (d + dd) * PS + cb);
                    const float4 s1 = *reinterpret_cast<const float4*>(sS + (d + dd) * PS + cb + 4);
                    fma8(P0, wv0[dd], s0, s1); fma8(P1, wv1[dd], s0, s1);
                    fma8(R0, qv0[dd], s0, s1); fma8(R1, qv1[dd], s0, s1);
                }
            }
            float4* d0 = reinterpret_cast<float4*>(sD + (2 * r2) * PS + cb);
            float4* d1 = reinterpret_cast<float4*>(sD + (2 * r2 + 1) * PS + cb);
            float4 u;
            u = d0[0]; d0[0] = make_float4(u.x - P0[0], u.y - P0[1], u.z - P0[2], u.w - P0[3]);
            u = d0[1]; d0[1] = make_float4(u.x - P0[4], u.y - P0[5], u.z - P0[6], u.w - P0[7]);
            u = d1[0]; d1[0] = make_float4(u.x - P1[0], u.y - P1[1], u.z - P1[2], u.w - P1[3]);
            u = d1[1]; d1[1] = make_float4(u.x - P1[4], u.y - P1[5], u.z - P1[6], u.w - P1[7]);
        }
        __syncthreads();
        // ---- O = R + QKd Delta (row 2 r2 sees s <= 2 r2, row 2 r2 + 1 one more)
        {
            const float* qk0 = sQK + (2 * r2) * 65;
            for (int s = 0; s <= 2 * r2 + 1; ++s) {
                const float4 s0 = *reinterpret_cast<const float4*>(sD + s * PS + cb), s1 = *reinterpret_cast<const float4*>(sD + s * PS + cb + 4);
                fma8(R0, qk0[s], s0, s1);            // QKd is zero above the diagonal
                fma8(R1, qk0[65 + s], s0, s1);
            }
            if (2 * r2 < C) {
                float* op = a.o + ((rowbase + 2 * r2) * Hv + h) * DV + c0 + cb;
                *reinterpret_cast<float4*>(op) = make_float4(R0[0], R0[1], R0[2], R0[3]);
                *reinterpret_cast<float4*>(op + 4) = make_float4(R0[4], R0[5], R0[6], R0[7]);
            }
            if (2 * r2 + 1 < C) {
                float* op = a.o + ((rowbase + 2 * r2 + 1) * Hv + h) * DV + c0 + cb;
                *reinterpret_cast<float4*>(op) = make_float4(R1[0], R1[1], R1[2], R1[3]);
                *reinterpret_cast<float4*>(op + 4) = make_float4(R1[4], R1[5], R1[6], R1[7]);
            }
        }
        // ---- S = D_C S0 + Kd^T Delta : thread -> state rows 4 d4 .. 4 d4 + 3, columns cb .. cb + 7
        for (int d4 = t / 8; d4 * 4 < DK; d4 += 32) {
            float acc[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 a0 = *reinterpret_cast<const float4*>(sS + (4 * d4 + i) * PS + cb);
                const float4 a1 = *reinterpret_cast<const float4*>(sS + (4 * d4 + i) * PS + cb + 4);
                acc[i][0] = DC * a0.x; acc[i][1] = DC * a0.y; acc[i][2] = DC * a0.z; acc[i][3] = DC * a0.w;
                acc[i][4] = DC * a1.x; acc[i][5] = DC * a1.y; acc[i][6] = DC * a1.z; acc[i][7] = DC * a1.w;
            }
#pragma unroll 2
            for (int s = 0; s < kChunk; ++s) {
                const float4 kv = *reinterpret_cast<const float4*>(sKd + s * PK + 4 * d4);
                const float4 s0 = *reinterpret_cast<const float4*>(sD + s * PS + cb), s1 = *reinterpret_cast<const float4*>(sD + s * PS + cb + 4);
                fma8(acc[0], kv.x, s0, s1); fma8(acc[1], kv.y, s0, s1); fma8(acc[2], kv.z, s0, s1); fma8(acc[3], kv.w, s0, s1);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                *reinterpret_cast<float4*>(sS + (4 * d4 + i) * PS + cb) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                *reinterpret_cast<float4*>(sS + (4 * d4 + i) * PS + cb + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
            }
        }
    }
    __syncthreads();
    for (int i = t; i < DK * kSlice / 4; i += 256) {
        const int d = (i * 4) / kSlice, c = (i * 4) % kSlice;
        *reinterpret_cast<float4*>(Sg + (size_t)d * DV + c0 + c) = *reinterpret_cast<const float4*>(sS + d * PS + c);
    }
}

// ---- tensor-core scan: the same three products on mma.sync m16n8k8 (TF32 operands, fp32 accumulation).
// The recurrent state lives in registers as accumulator fragments (warp w owns state rows 16w .. 16w+15, all
// 64 columns of the slice) and is never rounded; only the operand COPIES in shared memory are rounded to TF32
// (round-to-nearest, once, when they are stored).  Shared-memory pitches are chosen so that every fragment
// load is conflict-free: rows indexed by the fragment's group id use a pitch = 4 (mod 32), rows indexed by
// the k index a pitch = 8 (mod 32).
template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_chunk_scan_tc_kernel(const GdnScanArgs a) {
    constexpr int PA = DK + 4, PT = DK + 8, PS = kSlice + 8, PQ = kChunk + 4, NT = kSlice / 8;
    extern __shared__ __align__(16) float sm[];
    float* sW = sm;                          // [64][PA]   A operand, rows by group id
    float* sQd = sW + kChunk * PA;           // [64][PA]
    float* sKd = sQd + kChunk * PA;          // [64][PT]   read transposed (rows by k index)
    float* sS = sKd + kChunk * PT;           // [DK][PS]   B operand (TF32 copy of the state slice)
    float* sD = sS + DK * PS;                // [64][PS]   U slice, then Delta (B operand)
    float* sQK = sD + kChunk * PS;           // [64][PQ]   A operand

    const int slice = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, Hv = a.Hv, c0 = slice * kSlice;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const GdnSeqDesc2 sd = a.seqs[blockIdx.z];
    if (sd.n_rows <= a.min_rows || sd.slot < 0) return;
    PS_CHECK(PS_SLOT_OK(sd.slot) && PS_ROWS_OK(sd.row_start, sd.n_rows));
    int gc = 0;
    for (int s = 0; s < (int)blockIdx.z; ++s) {
        const GdnSeqDesc2 d = a.seqs[s];
        if (d.n_rows > a.min_rows && d.slot >= 0) gc += (d.n_rows + kChunk - 1) / kChunk;
    }
    float* Sg = a.state + ((size_t)sd.slot * Hv + h) * DK * DV;
    const bool own = warp < DK / 16;                    // this warp keeps state rows 16 warp .. 16 warp + 15
    const int mt = warp & 3, ch = warp >> 2;            // (a), (c): rows 16 mt .., columns 32 ch .. 32 ch + 31
    float S[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f; }
    if (own) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float2 lo = *reinterpret_cast<const float2*>(Sg + (size_t)(16 * warp + g) * DV + c0 + 8 * nt + 2 * t);
            const float2 hi = *reinterpret_cast<const float2*>(Sg + (size_t)(16 * warp + g + 8) * DV + c0 + 8 * nt + 2 * t);
            S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
            *reinterpret_cast<float2*>(sS + (16 * warp + g) * PS + 8 * nt + 2 * t) = make_float2(to_tf32(lo.x), to_tf32(lo.y));
            *reinterpret_cast<float2*>(sS + (16 * warp + g + 8) * PS + 8 * nt + 2 * t) = make_float2(to_tf32(hi.x), to_tf32(hi.y));
        }
    }

    // Tile traffic is asynchronous (cp.async, 16 bytes per copy; the preparation kernel already rounded W, Qd, Kd and
    // QKd to TF32).  Per chunk the copy groups are committed in the order [U] [QKd] [Kd] and, once product (a) has
    // released its operands, [W, Qd of the next chunk]; each product waits only for the groups it reads, so Kd and QKd
    // arrive under product (a) and the next chunk's W / Qd under products (c) and (d).
    auto cp16 = [](float* dst, const float* src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    };
    auto commit = []() { asm volatile("cp.async.commit_group;" ::: "memory"); };
    auto issue_wq = [&](int chunk_id) {
        const float* scr = a.scratch + ((size_t)chunk_id * Hv + h) * chunk_scratch_floats(DK, DV);
        const float* gW = scr; const float* gQd = gW + kChunk * DK;
        for (int i = tid; i < kChunk * DK / 4; i += 256) {
            const int r = (i * 4) / DK, d = (i * 4) % DK;
            cp16(sW + r * PA + d, gW + 4 * i);
            cp16(sQd + r * PA + d, gQd + 4 * i);
        }
    };
    issue_wq(gc);
    commit();

    for (int r0 = 0; r0 < sd.n_rows; r0 += kChunk, ++gc) {
        const int C = min(kChunk, sd.n_rows - r0);
        const size_t rowbase = (size_t)(sd.row_start + r0);
        const float* scr = a.scratch + ((size_t)gc * Hv + h) * chunk_scratch_floats(DK, DV);
        const float* gKd = scr + 2 * kChunk * DK;
        const float* gU = gKd + kChunk * DK; const float* gQK = gU + kChunk * DV;
        // the barrier that closed the previous chunk's product (d) released sD, sQK and sKd
        for (int i = tid; i < kChunk * kSlice / 4; i += 256) {
            const int r = (i * 4) / kSlice, c = (i * 4) % kSlice;
            cp16(sD + r * PS + c, gU + (size_t)r * DV + c0 + c);
        }
        commit();
        for (int i = tid; i < kChunk * kChunk / 4; i += 256) {
            const int r = (i * 4) / kChunk, c = (i * 4) % kChunk;
            cp16(sQK + r * PQ + c, gQK + 4 * i);
        }
        commit();
        for (int i = tid; i < kChunk * DK / 4; i += 256) {
            const int r = (i * 4) / DK, d = (i * 4) % DK;
            cp16(sKd + r * PT + d, gKd + 4 * i);
        }
        commit();
        const float DC = a.dc[(size_t)gc * Hv + h];
        asm volatile("cp.async.wait_group 2;" ::: "memory");      // [W, Qd] and [U] have landed (this thread's copies)
        __syncthreads();                                          // ... everyone's; also orders the sS stores before (a)
        // ---- (a) P = W S0, R = Qd S0 : rows 16 mt .., columns 32 ch + 8 nt ..
        float P[4][4], R[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) { P[nt][0] = P[nt][1] = P[nt][2] = P[nt][3] = 0.f; R[nt][0] = R[nt][1] = R[nt][2] = R[nt][3] = 0.f; }
        {
            const float* wr = sW + (16 * mt + g) * PA + t;
            const float* qr = sQd + (16 * mt + g) * PA + t;
#pragma unroll 4
            for (int ks = 0; ks < DK / 8; ++ks) {
                const float aw[4] = {wr[8 * ks], wr[8 * PA + 8 * ks], wr[8 * ks + 4], wr[8 * PA + 8 * ks + 4]};
                const float aq[4] = {qr[8 * ks], qr[8 * PA + 8 * ks], qr[8 * ks + 4], qr[8 * PA + 8 * ks + 4]};
                const float* sb = sS + (8 * ks + t) * PS + 32 * ch + g;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const float b0 = sb[8 * nt], b1 = sb[4 * PS + 8 * nt];
                    mma_tf32(P[nt], aw, b0, b1);
                    mma_tf32(R[nt], aq, b0, b1);
                }
            }
        }
        // Delta = U - P, written (TF32) over U in place: every lane owns its accumulator positions
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float* d0 = sD + (16 * mt + g) * PS + 32 * ch + 8 * nt + 2 * t;
            float* d1 = d0 + 8 * PS;
            const float2 u0 = *reinterpret_cast<const float2*>(d0), u1 = *reinterpret_cast<const float2*>(d1);
            *reinterpret_cast<float2*>(d0) = make_float2(to_tf32(u0.x - P[nt][0]), to_tf32(u0.y - P[nt][1]));
            *reinterpret_cast<float2*>(d1) = make_float2(to_tf32(u1.x - P[nt][2]), to_tf32(u1.y - P[nt][3]));
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");      // [QKd] has landed; [Kd] may still be in flight
        __syncthreads();                                          // Delta and QKd visible; (a) is done with sW / sQd
        if (r0 + kChunk < sd.n_rows) issue_wq(gc + 1);
        commit();                                                 // (an empty group on the last chunk keeps the counts uniform)
        // ---- (c) O = R + QKd Delta (QKd is zero above the diagonal: k-steps beyond this row tile are skipped)
        {
            const float* ar = sQK + (16 * mt + g) * PQ + t;
            for (int ks = 0; ks < 2 * mt + 2; ++ks) {
                const float aq[4] = {ar[8 * ks], ar[8 * PQ + 8 * ks], ar[8 * ks + 4], ar[8 * PQ + 8 * ks + 4]};
                const float* sb = sD + (8 * ks + t) * PS + 32 * ch + g;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) mma_tf32(R[nt], aq, sb[8 * nt], sb[4 * PS + 8 * nt]);
            }
            const int row_lo = 16 * mt + g, row_hi = row_lo + 8;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int col = c0 + 32 * ch + 8 * nt + 2 * t;
                if (row_lo < C) *reinterpret_cast<float2*>(a.o + ((rowbase + row_lo) * Hv + h) * DV + col) = make_float2(R[nt][0], R[nt][1]);
                if (row_hi < C) *reinterpret_cast<float2*>(a.o + ((rowbase + row_hi) * Hv + h) * DV + col) = make_float2(R[nt][2], R[nt][3]);
            }
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");      // [Kd] has landed; the next chunk's [W, Qd] may be in flight
        __syncthreads();
        // ---- (d) S = D_C S0 + Kd^T Delta : state rows 16 warp .., all columns; A[m = d][k = s] = Kd[s][d]
        if (own) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { S[nt][0] *= DC; S[nt][1] *= DC; S[nt][2] *= DC; S[nt][3] *= DC; }
            const float* kr = sKd + t * PT + 16 * warp + g;
#pragma unroll 2
            for (int ks = 0; ks < kChunk / 8; ++ks) {
                const float ak[4] = {kr[(8 * ks) * PT], kr[(8 * ks) * PT + 8], kr[(8 * ks + 4) * PT], kr[(8 * ks + 4) * PT + 8]};
                const float* sb = sD + (8 * ks + t) * PS + g;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_tf32(S[nt], ak, sb[8 * nt], sb[4 * PS + 8 * nt]);
            }
        }
        __syncthreads();                                 // (a) readers of sS and (c)/(d) readers of sD are done
        if (own) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                *reinterpret_cast<float2*>(sS + (16 * warp + g) * PS + 8 * nt + 2 * t) = make_float2(to_tf32(S[nt][0]), to_tf32(S[nt][1]));
                *reinterpret_cast<float2*>(sS + (16 * warp + g + 8) * PS + 8 * nt + 2 * t) = make_float2(to_tf32(S[nt][2]), to_tf32(S[nt][3]));
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    if (own) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            *reinterpret_cast<float2*>(Sg + (size_t)(16 * warp + g) * DV + c0 + 8 * nt + 2 * t) = make_float2(S[nt][0], S[nt][1]);
            *reinterpret_cast<float2*>(Sg + (size_t)(16 * warp + g + 8) * DV + c0 + 8 * nt + 2 * t) = make_float2(S[nt][2], S[nt][3]);
        }
    }
}

// One warp per (row, head): RMSNorm over the head's Dv outputs * SiLU(z).  E = Dv / 32 contiguous values per lane.
// grid = ceil(rows * Hv / 8), block = 256 threads
template <int E>
__global__ void __launch_bounds__(256) gdn_post_kernel(const float* o, const __nv_bfloat16* proj, int ld_proj, int z_off,
                                                       const __nv_bfloat16* norm_w, float eps, int Hv, int rows, const int* row_slot,
                                                       __nv_bfloat16* out, const GdnSeqDesc2* seqs, int n_seqs, int min_rows) {
    constexpr int Dv = 32 * E;
    const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= rows * Hv) return;
    const int row = item / Hv, h = item % Hv;
    if (row_slot[row] < 0 || !row_is_chunked(seqs, n_seqs, min_rows, row)) return;
    float v[E], z[E], w[E];
    const float* op = o + ((size_t)row * Hv + h) * Dv + lane * E;
    const __nv_bfloat16* zp = proj + (size_t)row * ld_proj + z_off + h * Dv + lane * E;
    if constexpr (E == 4) {
        const float4 f = *reinterpret_cast<const float4*>(op);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e) v[e] = op[e];
    }
#pragma unroll
    for (int e = 0; e < E; ++e) { z[e] = bf16_to_f32(zp[e]); w[e] = bf16_to_f32(norm_w[lane * E + e]); }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) ss = fmaf(v[e], v[e], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)Dv + eps);
    __nv_bfloat16* dst = out + (size_t)row * (Hv * Dv) + h * Dv + lane * E;
#pragma unroll
    for (int e = 0; e < E; e += 2)
        *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(v[e] * inv * w[e] * silu_f(z[e]), v[e + 1] * inv * w[e + 1] * silu_f(z[e + 1]));
}

}  // namespace ps

PS_DEFINE_LIMITS_SETTER(gdn_chunked)

// Floats of scratch needed for a step of `rows` rows in `n_seqs` sequences (upper bound on the chunks).
PS_API long long ps_gdn_chunked_scratch_floats(int rows, int n_seqs, int Hv, int Dk, int Dv) {
    const long long chunks = (rows + ps::kChunk - 1) / ps::kChunk + n_seqs;
    return chunks * Hv * (long long)ps::chunk_scratch_floats(Dk, Dv);
}

namespace ps {
template <int DK, int DV>
static int launch_chunked(const GdnPrepArgs& p, const GdnScanArgs& s, int max_chunks, cudaStream_t stream) {
    const size_t raw_b = (size_t)(kChunk + 3) * (2 * DK) * 2, at_b = sizeof(float) * (kChunk * 65 + kChunk * kTP + 3 * 16 * 17);
    const size_t smem_a = sizeof(float) * (2 * kChunk * (DK + 4) + 2 * kChunk) + (raw_b > at_b ? raw_b : at_b);
    const size_t smem_b = sizeof(float) * (3 * kChunk * (DK + 4) + DK * (kSlice + 4) + kChunk * (kSlice + 4) + kChunk * 65);
    const size_t smem_t = sizeof(float) * (2 * kChunk * (DK + 4) + kChunk * (DK + 8) + DK * (kSlice + 8) + kChunk * (kSlice + 8) +
                                           kChunk * (kChunk + 4));
    static bool set = false;
    static int use_tc = 1;
    if (!set) {
        cudaFuncSetAttribute(gdn_chunk_prep_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
        cudaFuncSetAttribute(gdn_chunk_scan_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b);
        cudaFuncSetAttribute(gdn_chunk_scan_tc_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_t);
        const char* e = getenv("PS_GDN_SCAN");            // "fp32": the CUDA-core scan (all-fp32 products)
        use_tc = (e == nullptr || e[0] != 'f') ? 1 : 0;
        set = true;
    }
    GdnPrepArgs pp = p;
    pp.round_tf32 = use_tc;
    gdn_chunk_prep_kernel<DK, DV><<<dim3(max_chunks, p.Hv), 256, smem_a, stream>>>(pp);
    int err = PS_LAUNCH_CHECK();
    if (err) return err;
    if (use_tc) gdn_chunk_scan_tc_kernel<DK, DV><<<dim3(DV / kSlice, p.Hv, p.n_seqs), 256, smem_t, stream>>>(s);
    else gdn_chunk_scan_kernel<DK, DV><<<dim3(DV / kSlice, p.Hv, p.n_seqs), 256, smem_b, stream>>>(s);
    return PS_LAUNCH_CHECK();
}
}  // namespace ps

// Chunked GDN mixer for prefill-sized steps.  `scratch` holds ps_gdn_chunked_scratch_floats() floats,
// `dc` one float per (chunk, head), `o` [rows, Hv, Dv] floats.
PS_API int ps_gdn_chunked(const void* proj, int ld_proj, int rows, int Hk, int Hv, int Dk, int Dv, const void* conv_w,
                          const void* A_log, const void* dt_bias, const void* norm_w, float eps, void* conv_state, int ring,
                          void* state, const void* seqs, int n_seqs, const void* row_slot, const void* row_pos,
                          int min_rows, void* scratch, void* dc, void* o, void* out, cudaStream_t stream) {
    using namespace ps;
    if (rows <= 0 || n_seqs <= 0 || Hk <= 0 || (Hv % Hk) || ring < 4) return (int)cudaErrorInvalidValue;
    GdnPrepArgs p;
    p.proj = (const __nv_bfloat16*)proj; p.ld_proj = ld_proj; p.Hk = Hk; p.Hv = Hv; p.Dk = Dk; p.Dv = Dv;
    p.conv_w = (const __nv_bfloat16*)conv_w; p.A_log = (const float*)A_log; p.dt_bias = (const float*)dt_bias;
    p.conv_state = (__nv_bfloat16*)conv_state; p.ring = ring; p.row_slot = (const int*)row_slot; p.row_pos = (const int*)row_pos;
    p.seqs = (const GdnSeqDesc2*)seqs; p.n_seqs = n_seqs; p.min_rows = min_rows; p.scratch = (float*)scratch; p.dc = (float*)dc;
    GdnScanArgs s;
    s.scratch = p.scratch; s.dc = p.dc; s.Hv = Hv; s.Dv = Dv; s.n_seqs = n_seqs; s.min_rows = min_rows; s.state = (float*)state; s.seqs = p.seqs;
    s.o = (float*)o;
    const int max_chunks = (rows + kChunk - 1) / kChunk + n_seqs;
    int err;
    if (Dk == 128 && Dv == 128) err = launch_chunked<128, 128>(p, s, max_chunks, stream);
    else if (Dk == 64 && Dv == 64) err = launch_chunked<64, 64>(p, s, max_chunks, stream);
    else return (int)cudaErrorInvalidValue;
    if (err) return err;
    gdn_history_kernel<<<dim3(Hv, ring, n_seqs), 128, 0, stream>>>(p);
    if ((err = PS_LAUNCH_CHECK())) return err;
    const int post_grid = (rows * Hv + 7) / 8, z_off = 2 * Hk * Dk + Hv * Dv;
    if (Dv == 128)
        gdn_post_kernel<4><<<post_grid, 256, 0, stream>>>((const float*)o, (const __nv_bfloat16*)proj, ld_proj, z_off, (const __nv_bfloat16*)norm_w,
                                                         eps, Hv, rows, (const int*)row_slot, (__nv_bfloat16*)out, p.seqs, n_seqs, min_rows);
    else
        gdn_post_kernel<2><<<post_grid, 256, 0, stream>>>((const float*)o, (const __nv_bfloat16*)proj, ld_proj, z_off, (const __nv_bfloat16*)norm_w,
                                                         eps, Hv, rows, (const int*)row_slot, (__nv_bfloat16*)out, p.seqs, n_seqs, min_rows);
    return PS_LAUNCH_CHECK();
}
