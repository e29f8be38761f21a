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

// ---- long prompts: the chunks of a sequence side by side ---------------------------------------------------------
// The loop above walks through a sequence's chunks one after the other, so a single long prompt keeps only
// (heads x value slices) blocks busy.  For prompts of more than one chunk the same sums are cut into three launches
// whose blocks are independent:
//   1. per chunk:    U_c = sum_j decay^(n-1-j) k_j v_j^T                                  (chunk_state_kernel)
//   2. per element:  S before chunk c, by the scan S <- decay^n S + U_c over the sequence's chunks; U_c is
//                    overwritten by the state BEFORE chunk c and the last S goes to the cache  (chunk_scan_kernel)
//   3. per chunk:    o_i = sum_j A[i][j] v_j + decay^(i+1) S_c^T q_i                         (chunk_out_kernel)
// Chunks are numbered through the batch (sequence after sequence); `w` below is that number.  Thread (ty, tx) of the
// 16 x 16 grid owns rows 4 ty .. 4 ty + 3 and columns 4 tx .. 4 tx + 3 of a product, and both operands of every
// product lie in shared memory so that its four values are one 16-byte load.
constexpr int PC = 64;           // tokens per chunk
constexpr int CP = PC + 4;       // row length of the transposed tiles ([dimension][token])

struct ChunkWork { int seq, slot, t0, n, pos0, first; };   // first: whether it is its sequence's first chunk

__device__ __forceinline__ bool chunk_work(const GfbBatch& b, int w, ChunkWork& c) {
    int left = w;
    for (int i = 0; i < b.n_seqs; i++) {
        const int q0 = b.cu_seqlens[i], qlen = b.cu_seqlens[i + 1] - q0;
        const int nc = (qlen + PC - 1) / PC;
        if (left < nc) {
            c.seq = i;
            c.slot = b.slots[i];
            c.t0 = q0 + left * PC;
            c.n = min(PC, qlen - left * PC);
            c.pos0 = b.lengths[c.slot] + left * PC;
            c.first = left == 0;
            return true;
        }
        left -= nc;
    }
    return false;
}

// (cos, sin) of pair u at position pos, or (1, 0) beyond the table (reported)
__device__ __forceinline__ float2 rot_of(const float* table, int table_len, int half, int pos, int u, int* status, int token) {
    if (pos >= 0 && pos < table_len) return make_float2(table[((size_t)pos * half + u) * 2], table[((size_t)pos * half + u) * 2 + 1]);
    if (u == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, token, pos);
    return make_float2(1.f, 0.f);
}

// VSX: value columns per block, 64 or 128 (a thread then owns two groups of four columns, 64 apart)
template <typename T, int VSX>
__global__ void __launch_bounds__(THREADS)
chunk_state_kernel(const T* __restrict__ src, int width, int k_off, int v_off, float* __restrict__ U, GfbBatch b,
                   const float* __restrict__ table, int table_len, int rot_dims, int pairing, const float* __restrict__ decay,
                   float k_scale, int H, int dk, int dv, int* status) {
    extern __shared__ __align__(16) float smem[];
    const int dk4 = (dk + 3) & ~3;
    float* Kc = smem;                               // [PC][dk4]: rotated k times its factor and decay^(n-1-j)
    float* Vs = Kc + (size_t)PC * dk4;              // [PC][VSX]
    float* pw = Vs + (size_t)PC * VSX;               // [PC+1]
    gfb_pdl_launch();
    const int w = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * VSX;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float dec = decay[h];
    for (int n = tid; n <= PC; n += THREADS) pw[n] = (float)pow((double)dec, (double)n);
    gfb_pdl_wait();
    ChunkWork c;
    if (!chunk_work(b, w, c)) return;
    __syncthreads();
    const int half = rot_dims >> 1, per_tok = dk4 - half;
    for (int e = tid; e < PC * per_tok; e += THREADS) {
        const int j = e / per_tok, u = e - j * per_tok;
        float* kd = Kc + (size_t)j * dk4;
        if (j >= c.n) {                              // rows beyond the chunk add nothing
            if (u < half) { kd[pairing == 1 ? u : 2 * u] = 0.f; kd[pairing == 1 ? u + half : 2 * u + 1] = 0.f; }
            else kd[rot_dims + (u - half)] = 0.f;
            continue;
        }
        const T* kh = src + (size_t)(c.t0 + j) * width + k_off + h * dk;
        const float f = k_scale * pw[c.n - 1 - j];
        if (u < half) {
            const float2 cs = rot_of(table, table_len, half, c.pos0 + j, u, status, c.t0 + j);
            const int i0 = pairing == 1 ? u : 2 * u, i1 = pairing == 1 ? u + half : 2 * u + 1;
            const float ka = gfb_to_f32(kh[i0]), kb = gfb_to_f32(kh[i1]);
            kd[i0] = (ka * cs.x - kb * cs.y) * f;
            kd[i1] = (kb * cs.x + ka * cs.y) * f;
        } else {
            const int i0 = rot_dims + (u - half);
            kd[i0] = i0 < dk ? gfb_to_f32(kh[i0]) * f : 0.f;
        }
    }
    for (int e = tid; e < PC * VSX; e += THREADS) {
        const int j = e / VSX, v = e - j * VSX;
        Vs[e] = (j < c.n && v0 + v < dv) ? gfb_to_f32(src[(size_t)(c.t0 + j) * width + v_off + h * dv + v0 + v]) : 0.f;
    }
    __syncthreads();
    float* Ug = U + ((size_t)w * H + h) * dk * dv;
    for (int d0 = 0; d0 < dk; d0 += 64) {
        if (d0 + 4 * ty >= dk4) continue;
        constexpr int NG = VSX / 64;
        float acc[NG][4][4];
#pragma unroll
        for (int g = 0; g < NG; g++)
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int cc = 0; cc < 4; cc++) acc[g][r][cc] = 0.f;
        for (int j = 0; j < c.n; j++) {
            const float4 k4 = *reinterpret_cast<const float4*>(Kc + (size_t)j * dk4 + d0 + 4 * ty);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
            for (int g = 0; g < NG; g++) {
                const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * VSX + 64 * g + 4 * tx);
                const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) acc[g][r][cc] = fmaf(kk[r], vv[cc], acc[g][r][cc]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int d = d0 + 4 * ty + r;
            if (d >= dk) continue;
#pragma unroll
            for (int g = 0; g < NG; g++)
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    const int v = v0 + 64 * g + 4 * tx + cc;
                    if (v < dv) Ug[(size_t)d * dv + v] = acc[g][r][cc];
                }
        }
    }
}

// One thread per element of a (sequence, head)'s state: U[c] <- S before chunk c, S <- decay^n S + U[c]; the last S is stored.
__global__ void __launch_bounds__(256)
chunk_scan_kernel(float* __restrict__ U, float* __restrict__ state, GfbBatch b, const float* __restrict__ decay, int H, int dk, int dv) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.y, h = blockIdx.z;
    const size_t per = (size_t)dk * dv;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    int first = 0;                                   // number of the sequence's first chunk
    for (int i = 0; i < s; i++) first += (b.cu_seqlens[i + 1] - b.cu_seqlens[i] + PC - 1) / PC;
    const int qlen = b.cu_seqlens[s + 1] - b.cu_seqlens[s];
    const int nc = (qlen + PC - 1) / PC;
    if (nc == 0) return;
    const float dec = decay[h];
    const float full = (float)pow((double)dec, (double)PC);
    const float last = (float)pow((double)dec, (double)(qlen - (nc - 1) * PC));
    float* Sg = state + ((size_t)b.slots[s] * H + h) * per + e;
    float S = *Sg;
    for (int c = 0; c < nc; c++) {
        float* u = U + ((size_t)(first + c) * H + h) * per + e;
        const float add = *u;
        *u = S;
        S = (c == nc - 1 ? last : full) * S + add;
    }
    *Sg = S;
}

// VSX: value columns per block, 64 or 128 (a thread then owns two groups of four columns, 64 apart)
template <typename T, int VSX>
__global__ void __launch_bounds__(THREADS)
chunk_out_kernel(const T* __restrict__ src, int width, int q_off, int k_off, int v_off, const float* __restrict__ U,
                 float* __restrict__ out, GfbBatch b, const float* __restrict__ table, int table_len, int rot_dims, int pairing,
                 const float* __restrict__ decay, float k_scale, int H, int dk, int dv, int* status) {
    extern __shared__ __align__(16) float smem[];
    float* Qt = smem;                               // [dk][CP]: rotated q, token fastest
    float* Kt = Qt + (size_t)dk * CP;               // [dk][CP]: rotated k times its factor
    float* Vs = Kt + (size_t)dk * CP;               // [PC][VSX]
    float* At = Vs + (size_t)PC * VSX;               // [PC][CP]: At[j][i] = (q_i . k_j) decay^(i-j) for j <= i
    float* Ss = At + (size_t)PC * CP;               // [dk][VSX]: the state before this chunk
    float* pw = Ss + (size_t)dk * VSX;               // [PC+1]
    gfb_pdl_launch();
    const int w = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * VSX;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float dec = decay[h];
    for (int n = tid; n <= PC; n += THREADS) pw[n] = (float)pow((double)dec, (double)n);
    gfb_pdl_wait();
    ChunkWork c;
    if (!chunk_work(b, w, c)) return;
    const int half = rot_dims >> 1, per_tok = dk - half;
    for (int e = tid; e < PC * per_tok; e += THREADS) {
        const int i = e / per_tok, u = e - i * per_tok;
        const bool live = i < c.n;
        const T* row = src + (size_t)(c.t0 + (live ? i : 0)) * width;
        const T* qh = row + q_off + h * dk;
        const T* kh = row + k_off + h * dk;
        if (u < half) {
            const int i0 = pairing == 1 ? u : 2 * u, i1 = pairing == 1 ? u + half : 2 * u + 1;
            float q0 = 0.f, q1 = 0.f, k0 = 0.f, k1 = 0.f;
            if (live) {
                const float2 cs = rot_of(table, table_len, half, c.pos0 + i, u, nullptr, 0);
                const float qa = gfb_to_f32(qh[i0]), qb = gfb_to_f32(qh[i1]), ka = gfb_to_f32(kh[i0]), kb = gfb_to_f32(kh[i1]);
                q0 = qa * cs.x - qb * cs.y; q1 = qb * cs.x + qa * cs.y;
                k0 = (ka * cs.x - kb * cs.y) * k_scale; k1 = (kb * cs.x + ka * cs.y) * k_scale;
            }
            Qt[(size_t)i0 * CP + i] = q0; Qt[(size_t)i1 * CP + i] = q1;
            Kt[(size_t)i0 * CP + i] = k0; Kt[(size_t)i1 * CP + i] = k1;
        } else {
            const int i0 = rot_dims + (u - half);
            Qt[(size_t)i0 * CP + i] = live ? gfb_to_f32(qh[i0]) : 0.f;
            Kt[(size_t)i0 * CP + i] = live ? gfb_to_f32(kh[i0]) * k_scale : 0.f;
        }
    }
    for (int e = tid; e < PC * VSX; e += THREADS) {
        const int j = e / VSX, v = e - j * VSX;
        Vs[e] = (j < c.n && v0 + v < dv) ? gfb_to_f32(src[(size_t)(c.t0 + j) * width + v_off + h * dv + v0 + v]) : 0.f;
    }
    const float* Ug = U + ((size_t)w * H + h) * dk * dv;
    for (int e = tid; e < dk * VSX; e += THREADS) {
        const int d = e / VSX, v = e - d * VSX;
        Ss[e] = (v0 + v < dv) ? Ug[(size_t)d * dv + v0 + v] : 0.f;
    }
    __syncthreads();
    {   // A, rows i = 4 ty + r, columns j = 4 tx + cc; stored transposed
        float acc[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int cc = 0; cc < 4; cc++) acc[r][cc] = 0.f;
        if (4 * tx <= 4 * ty + 3) {                    // tiles above the diagonal stay zero
            for (int d = 0; d < dk; d++) {
                const float4 q4 = *reinterpret_cast<const float4*>(Qt + (size_t)d * CP + 4 * ty);
                const float4 k4 = *reinterpret_cast<const float4*>(Kt + (size_t)d * CP + 4 * tx);
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) acc[r][cc] = fmaf(qq[r], kk[cc], acc[r][cc]);
            }
        }
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const int j = 4 * tx + cc;
            float a[4];
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int i = 4 * ty + r;
                a[r] = (j <= i && i < c.n) ? acc[r][cc] * pw[i - j] : 0.f;
            }
            *reinterpret_cast<float4*>(At + (size_t)j * CP + 4 * ty) = make_float4(a[0], a[1], a[2], a[3]);
        }
    }
    __syncthreads();
    if (4 * ty < c.n) {
        constexpr int NG = VSX / 64;
        float acc[NG][4][4], carry[NG][4][4];
#pragma unroll
        for (int g = 0; g < NG; g++)
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int cc = 0; cc < 4; cc++) { acc[g][r][cc] = 0.f; carry[g][r][cc] = 0.f; }
        const int jmax = min(c.n, 4 * ty + 4);           // A[i][j] = 0 beyond the row's own position
        for (int j = 0; j < jmax; j++) {
            const float4 a4 = *reinterpret_cast<const float4*>(At + (size_t)j * CP + 4 * ty);
            const float aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
            for (int g = 0; g < NG; g++) {
                const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * VSX + 64 * g + 4 * tx);
                const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) acc[g][r][cc] = fmaf(aa[r], vv[cc], acc[g][r][cc]);
            }
        }
        for (int d = 0; d < dk; d++) {
            const float4 q4 = *reinterpret_cast<const float4*>(Qt + (size_t)d * CP + 4 * ty);
            const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
            for (int g = 0; g < NG; g++) {
                const float4 s4 = *reinterpret_cast<const float4*>(Ss + d * VSX + 64 * g + 4 * tx);
                const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) carry[g][r][cc] = fmaf(qq[r], ss[cc], carry[g][r][cc]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int i = 4 * ty + r;
            if (i >= c.n) continue;
#pragma unroll
            for (int g = 0; g < NG; g++)
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    const int v = v0 + 64 * g + 4 * tx + cc;
                    if (v < dv) out[((size_t)(c.t0 + i) * H + h) * dv + v] = acc[g][r][cc] + pw[i + 1] * carry[g][r][cc];
                }
        }
    }
}

static size_t chunk_state_smem(int dk, int vs = VS) { return ((size_t)PC * ((dk + 3) & ~3) + (size_t)PC * vs + PC + 1) * sizeof(float); }
static size_t chunk_out_smem(int dk, int vs = VS) { return ((size_t)2 * dk * CP + (size_t)PC * vs + (size_t)PC * CP + (size_t)dk * vs + PC + 1) * sizeof(float); }

// Floats of scratch the three-launch form needs for a step of n_tokens tokens in n_seqs sequences (0: it does not apply).
GFB_API long gfb_retention_scratch_floats(int n_tokens, int n_seqs, int max_q_len, int H, int dk, int dv) {
    if (max_q_len <= PC || chunk_out_smem(dk) > 220 * 1024) return 0;
    return ((long)(n_tokens + PC - 1) / PC + n_seqs) * H * dk * dv;
}

// ---- decode steps: one token per sequence ------------------------------------------------------------------
// S <- decay S + k v^T and o = S^T q in one pass over the state, which is read and written once, straight from and to
// memory: thread (ty, tx) walks over key dimensions ty, ty + 16, ... with 4 value columns in a 16-byte access, all of
// a thread's loads independent of each other; the 16 partial outputs per column meet in shared memory and are added
// in ascending order.  For value heads whose size is a multiple of 4.
template <typename T>
__global__ void __launch_bounds__(THREADS)
retention_decode_kernel(const T* __restrict__ src, int width, int q_off, int k_off, int v_off, float* __restrict__ state,
                        float* __restrict__ out, GfbBatch b, const float* __restrict__ table, int table_len, int rot_dims,
                        int pairing, const float* __restrict__ decay, float k_scale, int H, int dk, int dv, int* status) {
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                               // [dk] rotated q
    float* ks = qs + dk;                            // [dk] rotated k times its factor
    float* red = ks + dk;                           // [16][VS]
    gfb_pdl_launch();
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * VS;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float dec = decay[h];
    const int slot = b.slots[s];
    const int t = b.cu_seqlens[s];
    gfb_pdl_wait();
    const int pos = b.lengths[slot];
    const T* row = src + (size_t)t * width;
    const int half = rot_dims >> 1;
    for (int u = tid; u < dk - half; u += THREADS) {
        const T* qh = row + q_off + h * dk;
        const T* kh = row + k_off + h * dk;
        if (u < half) {
            const float2 cs = rot_of(table, table_len, half, pos, u, (blockIdx.z == 0 && h == 0) ? status : nullptr, t);
            const int i0 = pairing == 1 ? u : 2 * u, i1 = pairing == 1 ? u + half : 2 * u + 1;
            const float qa = gfb_to_f32(qh[i0]), qb = gfb_to_f32(qh[i1]), ka = gfb_to_f32(kh[i0]), kb = gfb_to_f32(kh[i1]);
            qs[i0] = qa * cs.x - qb * cs.y; qs[i1] = qb * cs.x + qa * cs.y;
            ks[i0] = (ka * cs.x - kb * cs.y) * k_scale; ks[i1] = (kb * cs.x + ka * cs.y) * k_scale;
        } else {
            const int i0 = rot_dims + (u - half);
            qs[i0] = gfb_to_f32(qh[i0]);
            ks[i0] = gfb_to_f32(kh[i0]) * k_scale;
        }
    }
    const int col = v0 + 4 * tx;
    const bool live = col < dv;                     // dv % 4 == 0: a group of four columns is inside or outside
    float vv[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
#pragma unroll
        for (int c = 0; c < 4; c++) vv[c] = gfb_to_f32(row[v_off + h * dv + col + c]);
    }
    __syncthreads();
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        float* Sg = state + ((size_t)slot * H + h) * dk * dv + col;
#pragma unroll 4
        for (int d = ty; d < dk; d += 16) {
            float4 S4 = *reinterpret_cast<const float4*>(Sg + (size_t)d * dv);
            const float kd = ks[d], qd = qs[d];
            S4.x = dec * S4.x + kd * vv[0]; S4.y = dec * S4.y + kd * vv[1];
            S4.z = dec * S4.z + kd * vv[2]; S4.w = dec * S4.w + kd * vv[3];
            *reinterpret_cast<float4*>(Sg + (size_t)d * dv) = S4;
            o[0] = fmaf(S4.x, qd, o[0]); o[1] = fmaf(S4.y, qd, o[1]); o[2] = fmaf(S4.z, qd, o[2]); o[3] = fmaf(S4.w, qd, o[3]);
        }
    }
    *reinterpret_cast<float4*>(red + ty * VS + 4 * tx) = make_float4(o[0], o[1], o[2], o[3]);
    __syncthreads();
    if (tid < VS && v0 + tid < dv) {
        float acc = 0.f;
#pragma unroll
        for (int g = 0; g < 16; g++) acc += red[g * VS + tid];
        out[((size_t)t * H + h) * dv + v0 + tid] = acc;
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
                          const float* decay, float k_scale, int H, int dk, int dv, float* scratch, long scratch_floats,
                          int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (table == nullptr) rot_dims = 0;
    if (rot_dims % 2 || rot_dims > dk || rot_dims < 0) return gfb_fail("gfb_retention: %d rotated dimensions in a head of %d", rot_dims, dk);
    if (H > 65535) return gfb_fail("gfb_retention: %d heads exceed the grid", H);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const long need = gfb_retention_scratch_floats(n_tokens, n_seqs, max_q_len, H, dk, dv);
    if (need > 0 && scratch != nullptr && scratch_floats >= need) {
        // prompts of several chunks: the chunks side by side, in three launches
        const int n_chunks = (n_tokens + PC - 1) / PC + n_seqs;       // an upper bound; surplus blocks find no work
        if (n_chunks > 0x7fffffff / 2 || n_seqs > 65535) return gfb_fail("gfb_retention: too many chunks or sequences");
        // 128 value columns per block where the head has them and the tiles fit: the score tile is computed once per 128
        // columns and every 16-byte load of q, k or a score feeds 32 FMAs instead of 16
        const bool wide = dv >= 128 && chunk_out_smem(dk, 128) <= 220 * 1024;
        const int vs = wide ? 128 : VS;
        dim3 cgrid(n_chunks, H, (dv + vs - 1) / vs);
        const size_t s1 = chunk_state_smem(dk, vs), s3 = chunk_out_smem(dk, vs);
        cudaError_t e;
#define GO3(T, V)                                                                                                         \
        do {                                                                                                           \
            static bool configured = false;                                                                            \
            if (!configured) {                                                                                         \
                cudaFuncSetAttribute(chunk_state_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);  \
                cudaFuncSetAttribute(chunk_out_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);    \
                configured = true;                                                                                     \
            }                                                                                                          \
            e = gfb_launch(chunk_state_kernel<T, V>, cgrid, dim3(THREADS), s1, stream, (const T*)src, width, k_off, v_off, scratch, b, \
                           table, table_len, rot_dims, pairing, decay, k_scale, H, dk, dv, status);                    \
            if (e == cudaSuccess)                                                                                      \
                e = gfb_launch(chunk_scan_kernel, dim3((unsigned)(((size_t)dk * dv + 255) / 256), n_seqs, H), dim3(256), 0, stream, \
                               scratch, state, b, decay, H, dk, dv);                                                   \
            if (e == cudaSuccess)                                                                                      \
                e = gfb_launch(chunk_out_kernel<T, V>, cgrid, dim3(THREADS), s3, stream, (const T*)src, width, q_off, k_off, v_off, \
                               (const float*)scratch, out, b, table, table_len, rot_dims, pairing, decay, k_scale, H, dk, dv, status); \
        } while (0)
        if (dt == GFB_BF16 && wide) GO3(__nv_bfloat16, 128);
        else if (dt == GFB_BF16) GO3(__nv_bfloat16, 64);
        else if (dt == GFB_F32 && wide) GO3(float, 128);
        else if (dt == GFB_F32) GO3(float, 64);
        else return gfb_fail("gfb_retention: unknown type %d", dt);
#undef GO3
        return gfb_check(e, "gfb_retention (chunks side by side)");
    }
    dim3 grid(n_seqs, H, (dv + VS - 1) / VS);
    if (max_q_len == 1 && n_tokens == n_seqs && dv % 4 == 0 && ((uintptr_t)state & 15) == 0 && (size_t)(2 * dk + 16 * VS) * 4 <= 48 * 1024) {
        const size_t dsmem = (size_t)(2 * dk + 16 * VS) * sizeof(float);
        cudaError_t e;
        if (dt == GFB_BF16)
            e = gfb_launch(retention_decode_kernel<__nv_bfloat16>, grid, dim3(THREADS), dsmem, stream, (const __nv_bfloat16*)src, width,
                           q_off, k_off, v_off, state, out, b, table, table_len, rot_dims, pairing, decay, k_scale, H, dk, dv, status);
        else if (dt == GFB_F32)
            e = gfb_launch(retention_decode_kernel<float>, grid, dim3(THREADS), dsmem, stream, (const float*)src, width, q_off, k_off,
                           v_off, state, out, b, table, table_len, rot_dims, pairing, decay, k_scale, H, dk, dv, status);
        else
            return gfb_fail("gfb_retention: unknown type %d", dt);
        return gfb_check(e, "gfb_retention (decode)");
    }
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
