// Gated DeltaNet, row-sequential form: one launch covers the whole mixer between in_proj and out_proj.
//
// Per (sequence, value head) CTA, for each of the sequence's rows in order:
//   causal depthwise conv (kernel 4) + SiLU on this head's q/k/v channels, L2-normalise q (scaled by
//   Dk^-0.5) and k, beta = sigmoid(b), d = exp(-exp(A_log) * softplus(a + dt_bias)),
//   kv = (d S)^T k, delta = (v - kv) beta, S = d S + k (x) delta, o = S^T q,
//   out = RMSNorm_direct(o; w) * SiLU(z)  -> bf16.
// The fp32 state tile S[Dk, Dv] lives in registers for the whole launch, so decode reads and writes the
// state exactly once.  The reference spreads this over conv1d, silu, l2-normalise, scale, recurrence,
// per-group RMSNorm, silu and mul dispatches (src/phaseshift/models/qwen35/model/lower_to_primitives.cpp:
// 704-808; math in kernels/correctness/detail/gdn.inc:5-166).
//
// A row's arithmetic never depends on how many rows the launch carries, so verifying 1+K speculative
// rows reproduces K+1 single-row decodes bit for bit (the job of the reference's decode_rows_exact
// kernels, gdn/recurrence.hip:922-1190).  For speculative rollback the launch can write the new state
// to a second buffer and log (k, delta, d) per row; `ps_gdn_replay` re-applies an accepted prefix of
// that log to the untouched old state (the reference's compact-log commit, recurrence.hip:812-920).
//
// Conv history: [slots, Hv, ring, 2*Dk + Dv] bf16, slot (pos % ring) holds the pre-conv input of
// position pos.  Each value head keeps a private copy of its key head's q/k channels, so CTAs never
// share history and no ordering between them is needed; rolling back is just re-using an older pos.
#include "ps_common.cuh"

namespace ps {

struct GdnSeqDesc { int row_start; int n_rows; int slot; int pos_start; };

struct GdnArgs {
    const __nv_bfloat16* proj; int ld_proj;     // [rows, ld]: [q(Hk*Dk) | k(Hk*Dk) | v(Hv*Dv) | z(Hv*Dv) | b(Hv) | a(Hv)]
    int Hk, Hv;
    const __nv_bfloat16* conv_w;                // [2*Hk*Dk + Hv*Dv, 4]; tap 3 multiplies the current input
    const float* A_log; const float* dt_bias;   // [Hv]
    const __nv_bfloat16* norm_w; float eps;     // [Dv]
    __nv_bfloat16* conv_state; int ring;
    const float* state_in; float* state_out;    // [slots, Hv, Dk, Dv]
    const GdnSeqDesc* seqs;
    __nv_bfloat16* out;                         // [rows, Hv*Dv]
    float* log_k; float* log_delta; float* log_d;   // optional: [rows, Hv, Dk], [rows, Hv, Dv], [rows, Hv]
    // optional in-kernel beta/decay projections: b = xn . ba_w[h], a = xn . ba_w[Hv + h] (bf16 weights);
    // when null the kernel reads b and a from `proj`
    const __nv_bfloat16* ba_w; const __nv_bfloat16* xn; int ba_k;
    int max_rows;                               // sequences with more rows in this step belong to the chunked kernels
};

template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_rows_kernel(const GdnArgs a) {
    constexpr int CG = DV / 4;          // column groups of 4 consecutive columns
    constexpr int RG = 256 / CG;        // row groups
    constexpr int R = DK / RG;          // rows per thread
    constexpr int CH = 2 * DK + DV;     // conv channels owned by this head
    __shared__ float s_q[DK], s_k[DK], s_v[DV], s_red[32], s_red4[192];
    __shared__ float s_part[RG][DV], s_partq[RG][DV];
    __shared__ float s_vec[DV];

    const int h = blockIdx.x;
    const GdnSeqDesc sd = a.seqs[blockIdx.y];
    if (sd.n_rows <= 0 || sd.n_rows > a.max_rows) return;
    PS_CHECK(PS_SLOT_OK(sd.slot) && PS_ROWS_OK(sd.row_start, sd.n_rows) && sd.pos_start >= 0);
    const int hk = h / (a.Hv / a.Hk);
    const int t = threadIdx.x, cg = t % CG, rg = t / CG;
    const int q_off = hk * DK, k_off = a.Hk * DK + hk * DK, v_off = 2 * a.Hk * DK + h * DV;
    const int z_off = 2 * a.Hk * DK + a.Hv * DV + h * DV;
    const int b_off = 2 * a.Hk * DK + 2 * a.Hv * DV + h, a_off = b_off + a.Hv;

    cudaTriggerProgrammaticLaunchCompletion();
    float S[R][4];
    {
        // the recurrent state was last written by an earlier step, not by the stream predecessor
        const float* sp = a.state_in + ((size_t)sd.slot * a.Hv + h) * DK * DV;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float4 v = *reinterpret_cast<const float4*>(sp + (size_t)(rg + RG * r) * DV + cg * 4);
            S[r][0] = v.x; S[r][1] = v.y; S[r][2] = v.z; S[r][3] = v.w;
        }
    }
    cudaGridDependencySynchronize();
    __nv_bfloat16* hist = a.conv_state + ((size_t)sd.slot * a.Hv + h) * a.ring * CH;
    const float neg_expA = -__expf(a.A_log[h]);
    const float dtb = a.dt_bias[h];

    for (int r_i = 0; r_i < sd.n_rows; ++r_i) {
        const int row = sd.row_start + r_i, pos = sd.pos_start + r_i;
        const __nv_bfloat16* pr = a.proj + (size_t)row * a.ld_proj;
        // ---- conv + SiLU for this head's channels
        for (int c = t; c < CH; c += 256) {
            const int gc = c < DK ? q_off + c : (c < 2 * DK ? k_off + (c - DK) : v_off + (c - 2 * DK));
            const uint2 wraw = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)gc * 4);
            const float2 w01 = bf16x2_bits_to_f32x2(wraw.x), w23 = bf16x2_bits_to_f32x2(wraw.y);
            const __nv_bfloat16 xin = pr[gc];
            float taps[3];
#pragma unroll
            for (int j = 1; j <= 3; ++j) {
                float v = 0.f;
                if (pos - j >= 0) {
                    if (r_i - j >= 0) v = bf16_to_f32(a.proj[(size_t)(row - j) * a.ld_proj + gc]);
                    else v = bf16_to_f32(hist[(size_t)((pos - j) % a.ring) * CH + c]);
                }
                taps[j - 1] = v;   // taps[0] = x_{t-1}, taps[2] = x_{t-3}
            }
            float y = w01.x * taps[2];
            y = fmaf(w01.y, taps[1], y);
            y = fmaf(w23.x, taps[0], y);
            y = fmaf(w23.y, bf16_to_f32(xin), y);
            y = silu_f(y);
            if (c < DK) s_q[c] = y; else if (c < 2 * DK) s_k[c - DK] = y; else s_v[c - 2 * DK] = y;
        }
        __syncthreads();
        // history write happens after every thread has read its taps for this row
        for (int c = t; c < CH; c += 256) {
            const int gc = c < DK ? q_off + c : (c < 2 * DK ? k_off + (c - DK) : v_off + (c - 2 * DK));
            hist[(size_t)(pos % a.ring) * CH + c] = pr[gc];
        }
        // ---- L2 norms, k.q and (optionally) the beta / decay input projections: one fused block reduction
        float red5[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
        for (int i = t; i < DK; i += 256) { red5[0] += s_q[i] * s_q[i]; red5[1] += s_k[i] * s_k[i]; red5[4] += s_q[i] * s_k[i]; }
        if (a.ba_w != nullptr) {
            const __nv_bfloat16* xr = a.xn + (size_t)row * a.ba_k;
            const __nv_bfloat16* wb = a.ba_w + (size_t)h * a.ba_k;
            const __nv_bfloat16* wa = a.ba_w + (size_t)(a.Hv + h) * a.ba_k;
            for (int i = t * 2; i < a.ba_k; i += 512) {
                const float2 xv = bf16x2_bits_to_f32x2(*reinterpret_cast<const uint32_t*>(xr + i));
                const float2 bv = bf16x2_bits_to_f32x2(__ldg(reinterpret_cast<const uint32_t*>(wb + i)));
                const float2 av = bf16x2_bits_to_f32x2(__ldg(reinterpret_cast<const uint32_t*>(wa + i)));
                red5[2] = fmaf(xv.x, bv.x, red5[2]); red5[2] = fmaf(xv.y, bv.y, red5[2]);
                red5[3] = fmaf(xv.x, av.x, red5[3]); red5[3] = fmaf(xv.y, av.y, red5[3]);
            }
        }
        block_sum_n<5>(red5, s_red4);
        const float qn = rsqrtf(red5[0] + 1e-6f) * rsqrtf((float)DK);
        const float kn = rsqrtf(red5[1] + 1e-6f);
        const float kq = red5[4] * qn * kn;                       // k . q of the normalised vectors
        float b_in, a_in;
        if (a.ba_w != nullptr) {
            b_in = bf16_to_f32(f32_to_bf16(red5[2])); a_in = bf16_to_f32(f32_to_bf16(red5[3]));
        } else {
            b_in = bf16_to_f32(pr[b_off]); a_in = bf16_to_f32(pr[a_off]);
        }
        const float beta = sigmoid_f(b_in);
        const float gate = neg_expA * softplus_f(a_in + dtb);
        const float d = __expf(gate);
        // ---- one pass over the state: S <- d S, partial sums of S^T k and S^T q (both of the decayed old state)
        float kreg[R], qreg[R];
#pragma unroll
        for (int r = 0; r < R; ++r) { kreg[r] = s_k[rg + RG * r] * kn; qreg[r] = s_q[rg + RG * r] * qn; }
        float p[4] = {0.f, 0.f, 0.f, 0.f}, pq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int c = 0; c < 4; ++c) { S[r][c] *= d; p[c] = fmaf(S[r][c], kreg[r], p[c]); pq[c] = fmaf(S[r][c], qreg[r], pq[c]); }
        }
        *reinterpret_cast<float4*>(&s_part[rg][cg * 4]) = make_float4(p[0], p[1], p[2], p[3]);
        *reinterpret_cast<float4*>(&s_partq[rg][cg * 4]) = make_float4(pq[0], pq[1], pq[2], pq[3]);
        __syncthreads();
        // delta = beta (v - S^T k);  o = S_new^T q = S^T q + (k.q) delta   with S_new = S + k delta^T
        float ov = 0.f;
        if (t < DV) {
            float kv = 0.f, qv = 0.f;
#pragma unroll
            for (int g = 0; g < RG; ++g) { kv += s_part[g][t]; qv += s_partq[g][t]; }
            const float delta = (s_v[t] - kv) * beta;
            s_vec[t] = delta;
            ov = fmaf(kq, delta, qv);
            if (a.log_delta) a.log_delta[((size_t)row * a.Hv + h) * DV + t] = delta;
        }
        if (a.log_k) {
            for (int i = t; i < DK; i += 256) a.log_k[((size_t)row * a.Hv + h) * DK + i] = s_k[i] * kn;
            if (t == 0) a.log_d[(size_t)row * a.Hv + h] = d;
        }
        const float ss = block_sum(t < DV ? ov * ov : 0.f, s_red);      // its barriers also publish s_vec
        if (t < DV) {
            const float inv = rsqrtf(ss / (float)DV + a.eps);
            const float y = ov * inv * bf16_to_f32(a.norm_w[t]);
            const float z = bf16_to_f32(pr[z_off + t]);
            a.out[(size_t)row * (a.Hv * DV) + h * DV + t] = f32_to_bf16(y * silu_f(z));
        }
        // ---- S += k (x) delta (registers only)
        {
            const float4 dl = *reinterpret_cast<const float4*>(&s_vec[cg * 4]);
            const float dlr[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int c = 0; c < 4; ++c) S[r][c] = fmaf(kreg[r], dlr[c], S[r][c]);
            }
        }
        __syncthreads();      // s_q / s_k / s_v / s_part / s_vec are rewritten by the next row
    }
    {
        float* sp = a.state_out + ((size_t)sd.slot * a.Hv + h) * DK * DV;
#pragma unroll
        for (int r = 0; r < R; ++r)
            *reinterpret_cast<float4*>(sp + (size_t)(rg + RG * r) * DV + cg * 4) =
                make_float4(S[r][0], S[r][1], S[r][2], S[r][3]);
    }
}

struct GdnReplayArgs {
    float* state; int Hv;            // [slots, Hv, Dk, Dv]: old state, updated in place
    const GdnSeqDesc* seqs;          // n_rows = number of accepted rows to re-apply
    const float* log_k; const float* log_delta; const float* log_d;
};

// Re-apply S = d S + k (x) delta for the accepted rows; same expression order as the forward pass.
template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_replay_kernel(const GdnReplayArgs a) {
    constexpr int CG = DV / 4, RG = 256 / CG, R = DK / RG;
    const int h = blockIdx.x;
    const GdnSeqDesc sd = a.seqs[blockIdx.y];
    if (sd.n_rows <= 0) return;
    PS_CHECK(PS_SLOT_OK(sd.slot) && PS_ROWS_OK(sd.row_start, sd.n_rows));
    const int t = threadIdx.x, cg = t % CG, rg = t / CG;
    float* sp = a.state + ((size_t)sd.slot * a.Hv + h) * DK * DV;
    float S[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(sp + (size_t)(rg + RG * r) * DV + cg * 4);
        S[r][0] = v.x; S[r][1] = v.y; S[r][2] = v.z; S[r][3] = v.w;
    }
    for (int r_i = 0; r_i < sd.n_rows; ++r_i) {
        const size_t rh = (size_t)(sd.row_start + r_i) * a.Hv + h;
        const float d = a.log_d[rh];
        const float4 dl = *reinterpret_cast<const float4*>(a.log_delta + rh * DV + cg * 4);
        const float dlr[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float k = a.log_k[rh * DK + rg + RG * r];
#pragma unroll
            for (int c = 0; c < 4; ++c) { S[r][c] *= d; S[r][c] = fmaf(k, dlr[c], S[r][c]); }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
        *reinterpret_cast<float4*>(sp + (size_t)(rg + RG * r) * DV + cg * 4) = make_float4(S[r][0], S[r][1], S[r][2], S[r][3]);
}

}  // namespace ps

PS_DEFINE_LIMITS_SETTER(gdn_recurrent)

// Contract: the kernel may load the recurrent state of its slots BEFORE its stream predecessor has finished
// (programmatic dependent launch): the predecessor must therefore not write `state_in` of those slots.  Inside the
// engine that holds -- a projection kernel always sits between two GDN launches of one layer.  A caller that runs two
// ps_gdn_rows back to back on one slot and state buffer must put another kernel (or an event) between them, or set
// PS_PDL=0.
PS_API int ps_gdn_rows(const void* proj, int ld_proj, int Hk, int Hv, int Dk, int Dv, const void* conv_w,
                       const void* A_log, const void* dt_bias, const void* norm_w, float eps, void* conv_state,
                       int ring, const void* state_in, void* state_out, const void* seqs, int n_seqs, void* out,
                       void* log_k, void* log_delta, void* log_d, const void* ba_w, const void* xn, int ba_k, int max_rows,
                       cudaStream_t stream) {
    using namespace ps;
    if (n_seqs <= 0 || Hk <= 0 || (Hv % Hk) || ring < 4) return (int)cudaErrorInvalidValue;
    GdnArgs a;
    a.proj = (const __nv_bfloat16*)proj; a.ld_proj = ld_proj; a.Hk = Hk; a.Hv = Hv;
    a.conv_w = (const __nv_bfloat16*)conv_w; a.A_log = (const float*)A_log; a.dt_bias = (const float*)dt_bias;
    a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps; a.conv_state = (__nv_bfloat16*)conv_state; a.ring = ring;
    a.state_in = (const float*)state_in; a.state_out = (float*)state_out; a.seqs = (const GdnSeqDesc*)seqs;
    a.out = (__nv_bfloat16*)out; a.log_k = (float*)log_k; a.log_delta = (float*)log_delta; a.log_d = (float*)log_d;
    a.ba_w = (const __nv_bfloat16*)ba_w; a.xn = (const __nv_bfloat16*)xn; a.ba_k = ba_k;
    a.max_rows = max_rows > 0 ? max_rows : 0x7fffffff;
    if (ba_w != nullptr && (ba_k & 1)) return (int)cudaErrorInvalidValue;
    dim3 grid(Hv, n_seqs);
    if (Dk == 128 && Dv == 128) return launch_pdl(gdn_rows_kernel<128, 128>, grid, dim3(256), 0, stream, a);
    if (Dk == 64 && Dv == 64) return launch_pdl(gdn_rows_kernel<64, 64>, grid, dim3(256), 0, stream, a);
    return (int)cudaErrorInvalidValue;
}

PS_API int ps_gdn_replay(void* state, int Hv, int Dk, int Dv, const void* seqs, int n_seqs, const void* log_k,
                         const void* log_delta, const void* log_d, cudaStream_t stream) {
    using namespace ps;
    if (n_seqs <= 0) return (int)cudaErrorInvalidValue;
    GdnReplayArgs a;
    a.state = (float*)state; a.Hv = Hv; a.seqs = (const GdnSeqDesc*)seqs;
    a.log_k = (const float*)log_k; a.log_delta = (const float*)log_delta; a.log_d = (const float*)log_d;
    dim3 grid(Hv, n_seqs);
    if (Dk == 128 && Dv == 128) gdn_replay_kernel<128, 128><<<grid, 256, 0, stream>>>(a);
    else if (Dk == 64 && Dv == 64) gdn_replay_kernel<64, 64><<<grid, 256, 0, stream>>>(a);
    else return (int)cudaErrorInvalidValue;
    return PS_LAUNCH_CHECK();
}
