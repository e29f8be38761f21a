// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T        (S: [dk][dv] per head and sequence, 32-bit, zero at the start)
//     o_t = S_t^T q_t
//
// q and k are first rotated on their leading rot_dims dimensions by the token's position (pairs
// (i, i + rot_dims/2) or (2i, 2i+1)); k also takes a constant factor.  Everything behind the
// projections is 32-bit: rotation, decay powers, scores, state and outputs.
//
// The tokens a step brings for a sequence are taken C at a time.  With n tokens in a chunk, token
// i at distance i+1 from the state that was carried in:
//
//     A[i][j] = (q_i . k_j) * decay^(i-j)   for j <= i, else 0
//     o_i     = sum_j A[i][j] v_j  +  decay^(i+1) * S^T q_i
//     S       = decay^n * S  +  sum_j decay^(n-1-j) k_j v_j^T
//
// which is the recurrence written out, so a prompt may be cut anywhere and a decode step is the
// case n = 1.  One block per (sequence, head, slice of 64 value columns): the slices of a head are
// independent, each recomputes A.  The state slice lives in shared memory across the chunks and
// goes back to the cache's per-sequence state at the end.  Threads form a 16 x 16 grid, each
// owning a 4 x 4 tile of every product (rows ty + 16 r, columns tx + 16 c).
//
// gfb_retention_gate finishes a head: o / sqrt(mean(o^2) + eps) times silu(gate), to the compute type.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

constexpr int VS = 64;          // value columns per block
constexpr int THREADS = 256;

template <typename T, int C>
__global__ void __launch_bounds__(THREADS)
retention_kernel(const T* __restrict__ src, int width, int q_off, int k_off, int v_off, float* __restrict__ state,
                 float* __restrict__ out, GfbBatch b, const float* __restrict__ table, int table_len, int rot_dims,
                 int pairing, const float* __restrict__ decay, float k_scale, int H, int dk, int dv, int* status) {
    constexpr int RT = C / 16;                      // rows of a thread's tile over the chunk's tokens
    extern __shared__ float smem[];
    const int dkp = dk + 1;                         // padded row: the rows of a tile fall into different banks
    float* Qs = smem;                               // [C][dkp]
    float* Ks = Qs + (size_t)C * dkp;               // [C][dkp]
    float* Vs = Ks + (size_t)C * dkp;               // [C][VS]
    float* As = Vs + (size_t)C * VS;                // [C][C+1]
    float* Ss = As + (size_t)C * (C + 1);           // [dk][VS]
    float* pw = Ss + (size_t)dk * VS;               // [C+1]: decay^n
    gfb_pdl_launch();
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * VS;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float dec = decay[h];
    for (int n = tid; n <= C; n += THREADS) pw[n] = (float)pow((double)dec, (double)n);
    gfb_pdl_wait();
    const int slot = b.slots[s];
    const int t0 = b.cu_seqlens[s], t1 = b.cu_seqlens[s + 1];
    const int pos0 = b.lengths[slot];
    float* Sg = state + ((size_t)slot * H + h) * dk * dv;
    for (int e = tid; e < dk * VS; e += THREADS) {
        const int d = e / VS, v = e - d * VS;
        Ss[e] = (v0 + v < dv) ? Sg[(size_t)d * dv + v0 + v] : 0.f;
    }
    const int half = rot_dims >> 1;
    for (int c0 = t0; c0 < t1; c0 += C) {
        const int n = min(C, t1 - c0);
        __syncthreads();                            // the previous chunk is done with Qs, Ks, Vs, As; Ss is complete
        // q and k of the chunk, rotated; k with its factor.  One thread per (token, pair or passing element).
        const int per_tok = dk - half;              // `half` pairs + (dk - rot_dims) single elements
        for (int e = tid; e < n * per_tok; e += THREADS) {
            const int i = e / per_tok, u = e - i * per_tok;
            const int pos = pos0 + (c0 - t0) + i;
            const T* row = src + (size_t)(c0 + i) * width;
            const T* qh = row + q_off + h * dk;
            const T* kh = row + k_off + h * dk;
            float* qd = Qs + (size_t)i * dkp;
            float* kd = Ks + (size_t)i * dkp;
            if (u < half) {
                float cs = 1.f, sn = 0.f;
                if (pos >= 0 && pos < table_len) { cs = table[((size_t)pos * half + u) * 2]; sn = table[((size_t)pos * half + u) * 2 + 1]; }
                else if (u == 0 && blockIdx.z == 0 && h == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, c0 + i, pos);
                const int i0 = pairing == 1 ? u : 2 * u, i1 = pairing == 1 ? u + half : 2 * u + 1;
                const float qa = gfb_to_f32(qh[i0]), qb = gfb_to_f32(qh[i1]);
                const float ka = gfb_to_f32(kh[i0]), kb = gfb_to_f32(kh[i1]);
                qd[i0] = qa * cs - qb * sn;
                qd[i1] = qb * cs + qa * sn;
                kd[i0] = (ka * cs - kb * sn) * k_scale;
                kd[i1] = (kb * cs + ka * sn) * k_scale;
            } else {
                const int i0 = rot_dims + (u - half);
                qd[i0] = gfb_to_f32(qh[i0]);
                kd[i0] = gfb_to_f32(kh[i0]) * k_scale;
            }
        }
        for (int e = tid; e < C * VS; e += THREADS) {
            const int i = e / VS, v = e - i * VS;
            Vs[e] = (i < n && v0 + v < dv) ? gfb_to_f32(src[(size_t)(c0 + i) * width + v_off + h * dv + v0 + v]) : 0.f;
        }
        __syncthreads();
        // A = (Q K^T) with the decay of the distance, lower triangle
        {
            float acc[RT][RT];
#pragma unroll
            for (int r = 0; r < RT; r++)
#pragma unroll
                for (int c = 0; c < RT; c++) acc[r][c] = 0.f;
            if (ty < n && tx < n) {
                for (int d = 0; d < dk; d++) {
                    float qv[RT], kv[RT];
#pragma unroll
                    for (int r = 0; r < RT; r++) qv[r] = (ty + 16 * r < n) ? Qs[(size_t)(ty + 16 * r) * dkp + d] : 0.f;
#pragma unroll
                    for (int c = 0; c < RT; c++) kv[c] = (tx + 16 * c < n) ? Ks[(size_t)(tx + 16 * c) * dkp + d] : 0.f;
#pragma unroll
                    for (int r = 0; r < RT; r++)
#pragma unroll
                        for (int c = 0; c < RT; c++) acc[r][c] = fmaf(qv[r], kv[c], acc[r][c]);
                }
            }
#pragma unroll
            for (int r = 0; r < RT; r++)
#pragma unroll
                for (int c = 0; c < RT; c++) {
                    const int i = ty + 16 * r, j = tx + 16 * c;
                    As[(size_t)i * (C + 1) + j] = (j <= i && i < n) ? acc[r][c] * pw[i - j] : 0.f;
                }
        }
        __syncthreads();
        // o = A V + decay^(i+1) * Q S      (rows ty + 16 r, value columns tx + 16 c)
        {
            float acc[RT][4], carry[RT][4];
#pragma unroll
            for (int r = 0; r < RT; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) { acc[r][c] = 0.f; carry[r][c] = 0.f; }
            if (ty < n) {
                for (int j = 0; j < n; j++) {
                    float a[RT], vv[4];
#pragma unroll
                    for (int r = 0; r < RT; r++) a[r] = As[(size_t)(ty + 16 * r) * (C + 1) + j];
#pragma unroll
                    for (int c = 0; c < 4; c++) vv[c] = Vs[j * VS + tx + 16 * c];
#pragma unroll
                    for (int r = 0; r < RT; r++)
#pragma unroll
                        for (int c = 0; c < 4; c++) acc[r][c] = fmaf(a[r], vv[c], acc[r][c]);
                }
                for (int d = 0; d < dk; d++) {
                    float qv[RT], sv[4];
#pragma unroll
                    for (int r = 0; r < RT; r++) qv[r] = (ty + 16 * r < n) ? Qs[(size_t)(ty + 16 * r) * dkp + d] : 0.f;
#pragma unroll
                    for (int c = 0; c < 4; c++) sv[c] = Ss[d * VS + tx + 16 * c];
#pragma unroll
                    for (int r = 0; r < RT; r++)
#pragma unroll
                        for (int c = 0; c < 4; c++) carry[r][c] = fmaf(qv[r], sv[c], carry[r][c]);
                }
#pragma unroll
                for (int r = 0; r < RT; r++) {
                    const int i = ty + 16 * r;
                    if (i >= n) continue;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const int v = v0 + tx + 16 * c;
                        if (v < dv) out[((size_t)(c0 + i) * H + h) * dv + v] = acc[r][c] + pw[i + 1] * carry[r][c];
                    }
                }
            }
        }
        __syncthreads();                            // everyone has read S and K as they were
        for (int e = tid; e < n * dk; e += THREADS) {
            const int j = e / dk, d = e - j * dk;
            Ks[(size_t)j * dkp + d] *= pw[n - 1 - j];
        }
        __syncthreads();
        // S = decay^n S + K'^T V, 64 key dimensions at a time (rows ty + 16 r)
        for (int d0 = 0; d0 < dk; d0 += 64) {
            float acc[4][4];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[r][c] = 0.f;
            for (int j = 0; j < n; j++) {
                float kk[4], vv[4];
#pragma unroll
                for (int r = 0; r < 4; r++) kk[r] = (d0 + ty + 16 * r < dk) ? Ks[(size_t)j * dkp + d0 + ty + 16 * r] : 0.f;
#pragma unroll
                for (int c = 0; c < 4; c++) vv[c] = Vs[j * VS + tx + 16 * c];
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int c = 0; c < 4; c++) acc[r][c] = fmaf(kk[r], vv[c], acc[r][c]);
            }
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int d = d0 + ty + 16 * r;
                if (d >= dk) continue;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float* sp = Ss + d * VS + tx + 16 * c;
                    *sp = pw[n] * *sp + acc[r][c];
                }
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < dk * VS; e += THREADS) {
        const int d = e / VS, v = e - d * VS;
        if (v0 + v < dv) Sg[(size_t)d * dv + v0 + v] = Ss[e];
    }
}

static size_t retention_smem(int C, int dk) {
    return ((size_t)2 * C * (dk + 1) + (size_t)C * VS + (size_t)C * (C + 1) + (size_t)dk * VS + C + 1) * sizeof(float);
}

// src [T, width] of type dt holds q (H heads of dk) at q_off, k at k_off, v (H heads of dv) at v_off.
// state float32 [n_slots][H][dk][dv] is read and written for the batch's slots; out float32 [T][H][dv].
// table: float32 [table_len][rot_dims/2][2] (null or rot_dims 0: no rotation); decay float32 [H].
GFB_API int gfb_retention(const void* src, int dt, int width, int q_off, int k_off, int v_off, float* state, float* out,
                          const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths, int n_seqs,
                          int n_tokens, int max_q_len, const float* table, int table_len, int rot_dims, int pairing,
                          const float* decay, float k_scale, int H, int dk, int dv, int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (table == nullptr) rot_dims = 0;
    if (rot_dims % 2 || rot_dims > dk || rot_dims < 0) return gfb_fail("gfb_retention: %d rotated dimensions in a head of %d", rot_dims, dk);
    if (H > 65535) return gfb_fail("gfb_retention: %d heads exceed the grid", H);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    dim3 grid(n_seqs, H, (dv + VS - 1) / VS);
    // 64 tokens at a time where that fits beside the state slice; 16 for decode steps and very large heads
    const size_t limit = 220 * 1024;
    int C = (max_q_len > 16 && retention_smem(64, dk) <= limit) ? 64 : 16;
    const size_t smem = retention_smem(C, dk);
    if (smem > limit) return gfb_fail("gfb_retention: key heads of %d exceed the kernel's shared memory", dk);
    cudaError_t e;
#define GO(T, CC)                                                                                                      \
    do {                                                                                                               \
        static size_t allowed = 48 * 1024;                                                                             \
        if (smem > allowed) {                                                                                          \
            cudaFuncSetAttribute(retention_kernel<T, CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit);    \
            allowed = limit;                                                                                           \
        }                                                                                                              \
        e = gfb_launch(retention_kernel<T, CC>, grid, dim3(THREADS), smem, stream, (const T*)src, width, q_off, k_off, v_off, \
                       state, out, b, table, table_len, rot_dims, pairing, decay, k_scale, H, dk, dv, status);         \
    } while (0)
    if (dt == GFB_BF16 && C == 64) GO(__nv_bfloat16, 64);
    else if (dt == GFB_BF16) GO(__nv_bfloat16, 16);
    else if (dt == GFB_F32 && C == 64) GO(float, 64);
    else if (dt == GFB_F32) GO(float, 16);
    else return gfb_fail("gfb_retention: unknown type %d", dt);
#undef GO
    return gfb_check(e, "gfb_retention");
}

// out[t][h*dv + v] = o[t][h][v] / sqrt(mean_v(o[t][h]^2) + eps) * silu(gate[t][g_off + h*dv + v]); one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128)
retention_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int width, int g_off, T* __restrict__ out,
                      long items, int H, int dv, float eps) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= items) return;
    const long t = item / H;
    const int h = (int)(item - t * H);
    const float* row = o + (size_t)item * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) { const float x = row[i]; ss += x * x; }
    ss = gfb_warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    const T* g = gate + (size_t)t * width + g_off + (size_t)h * dv;
    T* dst = out + (size_t)item * dv;
    for (int i = lane; i < dv; i += 32) {
        const float z = gfb_to_f32(g[i]);
        dst[i] = gfb_from_f32<T>(row[i] * r * (z / (1.0f + expf(-z))));
    }
}

GFB_API int gfb_retention_gate(const float* o, const void* gate, int dt, int width, int g_off, void* out, int n_tokens, int H,
                               int dv, float eps, cudaStream_t stream) {
    const long items = (long)n_tokens * H;
    if (items <= 0) return 0;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(retention_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, (const __nv_bfloat16*)gate, width,
                       g_off, (__nv_bfloat16*)out, items, H, dv, eps);
    else if (dt == GFB_F32)
        e = gfb_launch(retention_gate_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, (const float*)gate, width, g_off,
                       (float*)out, items, H, dv, eps);
    else
        return gfb_fail("gfb_retention_gate: unknown type %d", dt);
    return gfb_check(e, "gfb_retention_gate");
}
