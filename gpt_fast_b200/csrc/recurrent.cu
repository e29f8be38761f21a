// Kernels of recurrent mixers whose state is a matrix per head, carried from token to token in 32-bit:
//
// gfb_short_conv    causal convolution over time per channel (a few taps, optional bias) and SiLU; the last
//                   taps - 1 inputs of every sequence are state, so a sequence may arrive in any portions
// gfb_ssd_scan      selective state space with a scalar decay per head and token:
//                       dt = softplus(dt_raw + dt_bias_h),  S <- exp(-exp(A_log_h) dt) S + dt B x^T,  y = S^T C + D_h x
// gfb_delta_rule    gated delta rule with a decay per head and key channel:
//                       S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                   with q, k made unit vectors per head (q also times dim^-1/2), beta = sigmoid(.),
//                   g = exp(-exp(A_log_h) softplus(a_raw + dt_bias))
// gfb_gated_norm    root-mean-square norm over groups of columns with a weight and a gate (SiLU or sigmoid) that
//                   is applied before or behind the norm
//
// The two recurrences share one layout: a block owns one (sequence, head) and walks through the sequence's
// tokens of this step; thread (column p, row group r) keeps RPT rows of column p of S in registers.  Sums over
// the rows are added per thread in ascending order and then over the row groups in ascending order, so a
// token's result is the same bits however the sequence was cut into steps or batched.  Everything is 32-bit.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float ldw(const void* p, int dt, size_t i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------ short convolution ----
constexpr int MAX_TAPS = 16;

// state of a slot: [taps - 1][C] inputs, oldest first, at state + slot * state_ld
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ src, int ld, int col_off, int C, const void* __restrict__ w,
                                  const void* __restrict__ bias, int w_dt, int taps, const float* __restrict__ state,
                                  size_t state_ld, float* __restrict__ out, GfbBatch b, int act) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = b.tok_seq[t];
    const int i = t - b.cu_seqlens[s];
    const float* st = state + (size_t)b.slots[s] * state_ld;
    float acc = bias != nullptr ? ldw(bias, w_dt, c) : 0.f;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;
        float v;
        if (i - back >= 0) v = gfb_to_f32(src[(size_t)(t - back) * ld + col_off + c]);
        else v = st[(size_t)(taps - 1 + i - back) * C + c];
        acc = fmaf(ldw(w, w_dt, (size_t)c * taps + j), v, acc);
    }
    out[(size_t)t * C + c] = act ? silu_f(acc) : acc;
}

template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ src, int ld, int col_off, int C, int taps, float* __restrict__ state,
                                  size_t state_ld, GfbBatch b) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int t0 = b.cu_seqlens[s], n = b.cu_seqlens[s + 1] - t0;
    float* st = state + (size_t)b.slots[s] * state_ld;
    float keep[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; k++) {
        if (k < taps - 1) {
            const int i = n - (taps - 1) + k;                   // index among this step's tokens; negative: older
            keep[k] = i >= 0 ? gfb_to_f32(src[(size_t)(t0 + i) * ld + col_off + c]) : st[(size_t)(taps - 1 + i) * C + c];
        }
    }
#pragma unroll
    for (int k = 0; k < MAX_TAPS; k++)
        if (k < taps - 1) st[(size_t)k * C + c] = keep[k];
}

// src [T, ld] of type dt, C channels from column col_off; w [C, taps] and bias [C] (or null) of type w_dt;
// state float32, slot stride state_ld, (taps - 1) * C numbers per slot; out float32 [T, C]; act: 1 = SiLU, 0 = none.
// The state is advanced by a second kernel behind the first.
GFB_API int gfb_short_conv(const void* src, int dt, int ld, int col_off, int C, const void* w, const void* bias, int w_dt,
                           int taps, float* state, long state_ld, float* out, const int* cu_seqlens, const int* tok_seq,
                           const int* slots, const int* lengths, int n_seqs, int n_tokens, int act, cudaStream_t stream) {
    if (n_tokens <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS) return gfb_fail("gfb_short_conv: %d taps (1 to %d)", taps, MAX_TAPS);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const int threads = 128;
    const unsigned cb = (unsigned)((C + threads - 1) / threads);
    if (cb > 65535) return gfb_fail("gfb_short_conv: %d channels exceed the grid limit", C);
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(short_conv_kernel<__nv_bfloat16>, dim3(n_tokens, cb), dim3(threads), 0, stream, (const __nv_bfloat16*)src, ld,
                       col_off, C, w, bias, w_dt, taps, (const float*)state, (size_t)state_ld, out, b, act);
    else if (dt == GFB_F32)
        e = gfb_launch(short_conv_kernel<float>, dim3(n_tokens, cb), dim3(threads), 0, stream, (const float*)src, ld, col_off, C, w,
                       bias, w_dt, taps, (const float*)state, (size_t)state_ld, out, b, act);
    else
        return gfb_fail("gfb_short_conv: unknown type %d", dt);
    if (gfb_check(e, "gfb_short_conv")) return 1;
    if (taps == 1) return 0;
    if (dt == GFB_BF16)
        e = gfb_launch(conv_state_kernel<__nv_bfloat16>, dim3(n_seqs, cb), dim3(threads), 0, stream, (const __nv_bfloat16*)src, ld,
                       col_off, C, taps, state, (size_t)state_ld, b);
    else
        e = gfb_launch(conv_state_kernel<float>, dim3(n_seqs, cb), dim3(threads), 0, stream, (const float*)src, ld, col_off, C, taps,
                       state, (size_t)state_ld, b);
    return gfb_check(e, "gfb_short_conv (state)");
}

// ------------------------------------------------------------------------------ the two recurrences ----
constexpr int TB = 8;                 // tokens whose inputs are staged in shared memory together

// sum over the row groups, ascending: part [RG][P] -> the column's total
__device__ __forceinline__ float sum_groups(const float* part, int RG, int P, int p) {
    float v = part[p];
    for (int r = 1; r < RG; r++) v += part[(size_t)r * P + p];
    return v;
}

// x [T, ldx] float32: head h's P inputs at column h * P, group g's N numbers of B at b_off + g * N, of C at
// c_off + g * N.  dt_raw: [T, ld_dt] of type TD, head h at column dt_off + h.
template <typename TD, int RPT>
__global__ void __launch_bounds__(RPT == 16 ? 1024 : RPT == 128 ? 256 : 512)
ssd_scan_kernel(const float* __restrict__ x, int ldx, int b_off, int c_off, const TD* __restrict__ dt_raw, int ld_dt,
                                int dt_off, const void* __restrict__ dt_bias, const void* __restrict__ a_log,
                                const void* __restrict__ skip, int w_dt, float* __restrict__ state, size_t state_ld,
                                float* __restrict__ out, GfbBatch b, int H, int P, int N, int G) {
    extern __shared__ float sm[];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int RG = (N + RPT - 1) / RPT;
    float* sB = sm;                       // [TB][N]
    float* sC = sB + TB * N;              // [TB][N]
    float* sX = sC + TB * N;              // [TB][P]
    float* sDt = sX + TB * P;             // [TB]
    float* sA = sDt + TB;                 // [TB]
    float* part = sA + TB;                // [TB][RG][P]
    const int tid = threadIdx.x;
    const bool active = tid < P * RG;
    const int p = active ? tid % P : 0, rg = active ? tid / P : 0;
    const int t0 = b.cu_seqlens[s], t1 = b.cu_seqlens[s + 1];
    float* S = state + (size_t)b.slots[s] * state_ld + (size_t)h * N * P;
    float st[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int n = rg * RPT + r;
        st[r] = (active && n < N) ? S[(size_t)n * P + p] : 0.f;
    }
    const float bias = ldw(dt_bias, w_dt, h), rate = expf(ldw(a_log, w_dt, h)), dskip = skip != nullptr ? ldw(skip, w_dt, h) : 0.f;
    for (int tile = t0; tile < t1; tile += TB) {
        const int nt = min(TB, t1 - tile);
        __syncthreads();                                       // the previous tile's reads are done
        for (int i = tid; i < nt * N; i += blockDim.x) {
            const int tt = i / N, n = i - tt * N;
            const float* row = x + (size_t)(tile + tt) * ldx;
            sB[tt * N + n] = row[b_off + g * N + n];
            sC[tt * N + n] = row[c_off + g * N + n];
        }
        for (int i = tid; i < nt * P; i += blockDim.x) {
            const int tt = i / P, q = i - tt * P;
            sX[tt * P + q] = x[(size_t)(tile + tt) * ldx + (size_t)h * P + q];
        }
        if (tid < nt) {
            const float d = softplus_f(gfb_to_f32(dt_raw[(size_t)(tile + tid) * ld_dt + dt_off + h]) + bias);
            sDt[tid] = d;
            sA[tid] = expf(-rate * d);
        }
        __syncthreads();
        if (active) {
            for (int tt = 0; tt < nt; tt++) {
                const float a = sA[tt], dx = sDt[tt], xp = sX[tt * P + p];
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const int n = rg * RPT + r;
                    if (n < N) {
                        st[r] = fmaf(a, st[r], (dx * sB[tt * N + n]) * xp);
                        acc = fmaf(st[r], sC[tt * N + n], acc);
                    }
                }
                part[((size_t)tt * RG + rg) * P + p] = acc;
            }
        }
        __syncthreads();
        for (int i = tid; i < nt * P; i += blockDim.x) {
            const int tt = i / P, q = i - tt * P;
            out[(size_t)(tile + tt) * H * P + (size_t)h * P + q] = sum_groups(part + (size_t)tt * RG * P, RG, P, q) + dskip * sX[tt * P + q];
        }
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            const int n = rg * RPT + r;
            if (n < N) S[(size_t)n * P + p] = st[r];
        }
    }
}

// qkv [T, ldq] float32 (convolved, activated): query head j at q_off + j * d, key head j at k_off + j * d, value head
// h at v_off + h * dv.  beta_raw [T, ld_b] of type TD, head h at column beta_off + h.  a_raw [T, ld_a] float32, head
// h's d channels at a_off + h * d; dt_bias [H * d].
template <typename TD, int RPT>
__global__ void __launch_bounds__(RPT == 16 ? 1024 : RPT == 128 ? 256 : 512)
delta_rule_kernel(const float* __restrict__ qkv, int ldq, int q_off, int k_off, int v_off,
                                  const TD* __restrict__ beta_raw, int ld_b, int beta_off, const float* __restrict__ a_raw, int ld_a,
                                  int a_off, const void* __restrict__ dt_bias, const void* __restrict__ a_log, int w_dt,
                                  float* __restrict__ state, size_t state_ld, float* __restrict__ out, GfbBatch b, int H, int KH,
                                  int d, int dv, float q_scale, float unit_eps) {
    extern __shared__ float sm[];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, kh = h / (H / KH);
    const int RG = (d + RPT - 1) / RPT;
    float* sQ = sm;                       // [TB][d]
    float* sK = sQ + TB * d;              // [TB][d]
    float* sG = sK + TB * d;              // [TB][d]
    float* sV = sG + TB * d;              // [TB][dv]
    float* sBeta = sV + TB * dv;          // [TB]
    float* part1 = sBeta + TB;            // [2][RG][dv]
    float* part2 = part1 + 2 * RG * dv;   // [TB][RG][dv]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const bool active = tid < dv * RG;
    const int p = active ? tid % dv : 0, rg = active ? tid / dv : 0;
    const int t0 = b.cu_seqlens[s], t1 = b.cu_seqlens[s + 1];
    float* S = state + (size_t)b.slots[s] * state_ld + (size_t)h * d * dv;
    float st[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int i = rg * RPT + r;
        st[r] = (active && i < d) ? S[(size_t)i * dv + p] : 0.f;
    }
    const float rate = expf(ldw(a_log, w_dt, h));
    for (int tile = t0; tile < t1; tile += TB) {
        const int nt = min(TB, t1 - tile);
        __syncthreads();
        for (int i = tid; i < nt * d; i += blockDim.x) {
            const int tt = i / d, c = i - tt * d;
            const float* row = qkv + (size_t)(tile + tt) * ldq;
            sQ[tt * d + c] = row[q_off + kh * d + c];
            sK[tt * d + c] = row[k_off + kh * d + c];
            const float a = a_raw[(size_t)(tile + tt) * ld_a + a_off + (size_t)h * d + c] + ldw(dt_bias, w_dt, (size_t)h * d + c);
            sG[tt * d + c] = expf(-rate * softplus_f(a));
        }
        for (int i = tid; i < nt * dv; i += blockDim.x) {
            const int tt = i / dv, c = i - tt * dv;
            sV[tt * dv + c] = qkv[(size_t)(tile + tt) * ldq + v_off + (size_t)h * dv + c];
        }
        if (tid < nt) sBeta[tid] = sigmoid_f(gfb_to_f32(beta_raw[(size_t)(tile + tid) * ld_b + beta_off + h]));
        __syncthreads();
        // unit vectors: a warp per (token, q or k); lanes add strided squares, a fixed tree adds the lanes
        for (int item = warp; item < 2 * nt; item += nwarp) {
            float* vec = (item & 1 ? sK : sQ) + (item >> 1) * d;
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) ss = fmaf(vec[c], vec[c], ss);
            ss = gfb_warp_sum(ss);
            const float f = (1.0f / sqrtf(ss + unit_eps)) * (item & 1 ? 1.0f : q_scale);
            for (int c = lane; c < d; c += 32) vec[c] *= f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            float* p1 = part1 + (size_t)(tt & 1) * RG * dv;
            float acc = 0.f;
            if (active) {
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const int i = rg * RPT + r;
                    if (i < d) {
                        st[r] *= sG[tt * d + i];
                        acc = fmaf(st[r], sK[tt * d + i], acc);
                    }
                }
                if (RG > 1) p1[(size_t)rg * dv + p] = acc;
            }
            if (RG > 1) {
                __syncthreads();
                if (active) acc = sum_groups(p1, RG, dv, p);
            }
            if (active) {
                const float u = sBeta[tt] * (sV[tt * dv + p] - acc);
                float o = 0.f;
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const int i = rg * RPT + r;
                    if (i < d) {
                        st[r] = fmaf(sK[tt * d + i], u, st[r]);
                        o = fmaf(st[r], sQ[tt * d + i], o);
                    }
                }
                part2[((size_t)tt * RG + rg) * dv + p] = o;
            }
        }
        __syncthreads();
        for (int i = tid; i < nt * dv; i += blockDim.x) {
            const int tt = i / dv, c = i - tt * dv;
            out[(size_t)(tile + tt) * H * dv + (size_t)h * dv + c] = sum_groups(part2 + (size_t)tt * RG * dv, RG, dv, c);
        }
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            const int i = rg * RPT + r;
            if (i < d) S[(size_t)i * dv + p] = st[r];
        }
    }
}

// rows per thread for a state of `rows` x `cols`: the fewest whose block fits its thread limit; 0 if none does
static int pick_rpt(int rows, int cols, int* threads) {
    const int rpt[4] = {16, 32, 64, 128}, limit[4] = {1024, 512, 512, 256};
    for (int i = 0; i < 4; i++) {
        const int need = cols * ((rows + rpt[i] - 1) / rpt[i]);
        if (need <= limit[i]) {
            *threads = (need + 31) / 32 * 32;
            return rpt[i];
        }
    }
    return 0;
}

template <typename K>
static int allow_smem(K kernel, size_t smem, const char* what) {
    if (smem > 200 * 1024) return gfb_fail("%s: %zu bytes of shared memory", what, smem);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gfb_fail("%s: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

// state float32: slot stride state_ld, per slot [H][N][P]; out float32 [T, H, P]; vectors dt_bias, a_log, skip [H] of w_dt
// (skip may be null); dt_raw of type dt_dt.
GFB_API int gfb_ssd_scan(const float* x, int ldx, int b_off, int c_off, const void* dt_raw, int dt_dt, int ld_dt, int dt_off,
                         const void* dt_bias, const void* a_log, const void* skip, int w_dt, float* state, long state_ld,
                         float* out, const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                         int n_seqs, int n_tokens, int H, int P, int N, int G, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (G <= 0 || H % G) return gfb_fail("gfb_ssd_scan: %d heads do not divide into %d groups", H, G);
    if (H > 65535) return gfb_fail("gfb_ssd_scan: %d heads exceed the grid limit", H);
    int threads = 0;
    const int rpt = pick_rpt(N, P, &threads);
    if (!rpt) return gfb_fail("gfb_ssd_scan: a state of %d x %d per head does not fit a block", N, P);
    const int RG = (N + rpt - 1) / rpt;
    const size_t smem = ((size_t)TB * (2 * N + P + 2) + (size_t)TB * RG * P) * sizeof(float);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    cudaError_t e = cudaSuccess;
#define GO(TD, R)                                                                                                          \
    do {                                                                                                                   \
        if (allow_smem(ssd_scan_kernel<TD, R>, smem, "gfb_ssd_scan")) return 1;                                            \
        e = gfb_launch(ssd_scan_kernel<TD, R>, dim3(n_seqs, H), dim3(threads), smem, stream, x, ldx, b_off, c_off, (const TD*)dt_raw, \
                       ld_dt, dt_off, dt_bias, a_log, skip, w_dt, state, (size_t)state_ld, out, b, H, P, N, G);            \
    } while (0)
#define PICK(TD) do { if (rpt == 16) GO(TD, 16); else if (rpt == 32) GO(TD, 32); else if (rpt == 64) GO(TD, 64); else GO(TD, 128); } while (0)
    if (dt_dt == GFB_BF16) PICK(__nv_bfloat16);
    else if (dt_dt == GFB_F32) PICK(float);
    else return gfb_fail("gfb_ssd_scan: unknown type %d", dt_dt);
#undef PICK
#undef GO
    return gfb_check(e, "gfb_ssd_scan");
}

// state float32: slot stride state_ld, per slot [H][d][dv]; out float32 [T, H, dv]; dt_bias [H * d], a_log [H] of w_dt.
GFB_API int gfb_delta_rule(const float* qkv, int ldq, int q_off, int k_off, int v_off, const void* beta_raw, int b_dt, int ld_b,
                           int beta_off, const float* a_raw, int ld_a, int a_off, const void* dt_bias, const void* a_log, int w_dt,
                           float* state, long state_ld, float* out, const int* cu_seqlens, const int* tok_seq, const int* slots,
                           const int* lengths, int n_seqs, int n_tokens, int H, int KH, int d, int dv, float q_scale,
                           float unit_eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (KH <= 0 || H % KH) return gfb_fail("gfb_delta_rule: %d heads do not divide into %d query/key heads", H, KH);
    if (H > 65535) return gfb_fail("gfb_delta_rule: %d heads exceed the grid limit", H);
    int threads = 0;
    const int rpt = pick_rpt(d, dv, &threads);
    if (!rpt) return gfb_fail("gfb_delta_rule: a state of %d x %d per head does not fit a block", d, dv);
    const int RG = (d + rpt - 1) / rpt;
    const size_t smem = ((size_t)TB * (3 * d + dv + 1) + (size_t)(2 + TB) * RG * dv) * sizeof(float);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    cudaError_t e = cudaSuccess;
#define GO(TD, R)                                                                                                          \
    do {                                                                                                                   \
        if (allow_smem(delta_rule_kernel<TD, R>, smem, "gfb_delta_rule")) return 1;                                        \
        e = gfb_launch(delta_rule_kernel<TD, R>, dim3(n_seqs, H), dim3(threads), smem, stream, qkv, ldq, q_off, k_off, v_off,   \
                       (const TD*)beta_raw, ld_b, beta_off, a_raw, ld_a, a_off, dt_bias, a_log, w_dt, state, (size_t)state_ld, \
                       out, b, H, KH, d, dv, q_scale, unit_eps);                                                           \
    } while (0)
#define PICK(TD) do { if (rpt == 16) GO(TD, 16); else if (rpt == 32) GO(TD, 32); else if (rpt == 64) GO(TD, 64); else GO(TD, 128); } while (0)
    if (b_dt == GFB_BF16) PICK(__nv_bfloat16);
    else if (b_dt == GFB_F32) PICK(float);
    else return gfb_fail("gfb_delta_rule: unknown type %d", b_dt);
#undef PICK
#undef GO
    return gfb_check(e, "gfb_delta_rule");
}

// ------------------------------------------------------------------------------ gated group norm ----
// One warp per (token, group of `gs` columns): v = y, times act(gate) first if gate_first; n = v / sqrt(mean(v^2) + eps)
// * weight[col % w_len]; times act(gate) behind the norm otherwise.  act: 0 = SiLU, 1 = sigmoid.
template <typename TG, typename TO>
__global__ void gated_norm_kernel(const float* __restrict__ y, const TG* __restrict__ gate, int ld_gate, int gate_off,
                                  const void* __restrict__ weight, int w_dt, int w_len, TO* __restrict__ out, int T, int groups,
                                  int gs, float eps, int act, int gate_first) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)T * groups) return;
    const int t = (int)(item / groups), g = (int)(item - (long)t * groups);
    const float* yr = y + ((size_t)t * groups + g) * gs;
    const TG* gr = gate + (size_t)t * ld_gate + gate_off + (size_t)g * gs;
    float ss = 0.f;
    for (int c = lane; c < gs; c += 32) {
        float v = yr[c];
        if (gate_first) { const float z = gfb_to_f32(gr[c]); v *= act ? sigmoid_f(z) : silu_f(z); }
        ss = fmaf(v, v, ss);
    }
    ss = gfb_warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)gs + eps);
    TO* o = out + ((size_t)t * groups + g) * gs;
    for (int c = lane; c < gs; c += 32) {
        float v = yr[c];
        const float z = gfb_to_f32(gr[c]);
        const float a = act ? sigmoid_f(z) : silu_f(z);
        if (gate_first) v *= a;
        v = v * r * ldw(weight, w_dt, (size_t)(g * gs + c) % w_len);
        if (!gate_first) v *= a;
        o[c] = gfb_from_f32<TO>(v);
    }
}

// y float32 [T, groups * gs]; gate [T, ld_gate] of gate_dt, its groups * gs columns from gate_off; weight [w_len] of
// w_dt, indexed by column mod w_len; out [T, groups * gs] of out_dt.
GFB_API int gfb_gated_norm(const float* y, const void* gate, int gate_dt, int ld_gate, int gate_off, const void* weight, int w_dt,
                           int w_len, void* out, int out_dt, int T, int groups, int gs, float eps, int act, int gate_first,
                           cudaStream_t stream) {
    if (T <= 0 || groups <= 0 || gs <= 0) return 0;
    if (w_len <= 0) return gfb_fail("gfb_gated_norm: a weight of %d numbers", w_len);
    const long items = (long)T * groups;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
#define GO(TG, TO) e = gfb_launch(gated_norm_kernel<TG, TO>, dim3(blocks), dim3(128), 0, stream, y, (const TG*)gate, ld_gate, gate_off, \
                                  weight, w_dt, w_len, (TO*)out, T, groups, gs, eps, act, gate_first)
    if (gate_dt == GFB_BF16 && out_dt == GFB_BF16) GO(bf16, bf16);
    else if (gate_dt == GFB_F32 && out_dt == GFB_BF16) GO(float, bf16);
    else if (gate_dt == GFB_F32 && out_dt == GFB_F32) GO(float, float);
    else if (gate_dt == GFB_BF16 && out_dt == GFB_F32) GO(bf16, float);
    else return gfb_fail("gfb_gated_norm: unsupported types gate %d out %d", gate_dt, out_dt);
#undef GO
    return gfb_check(e, "gfb_gated_norm");
}
