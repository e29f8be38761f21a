// Kernels of latent attention: keys and values of all heads are expanded from one normed latent vector
// c [rank] per token, and one rotated key part k_r [rot] per token is shared by all heads.  Only (c, k_r) is
// cached, as one "key row" of rank + rot numbers.  Because the expansion is linear, attention runs on the
// latent itself:
//
//     score_h(i, j) = scale * ( (W_uk,h^T q_h,i) . c_j  +  rot(q_r,h,i) . rot(k_r,j) )
//     y_h,i         = W_uv,h  sum_j p_h(i, j) c_j
//
// gfb_latent_prepare   per token: c = rms_norm(first `rank` outputs of the down projection) * weight, the last
//                      `rot` outputs rotated by the token's position; both appended to the cache as one row;
//                      every head's rotated query part turned and written behind the head's latent query.
// gfb_headwise_linear  out[t, h, :] = W_h in[t, h, :] with a weight per head (the two expansions above), strided
//                      inputs and outputs, optionally times sigmoid(gate[t, h, :]).
// Norm, angles and rotation are 32-bit; sums are 32-bit in a fixed order.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float ld_any(const void* p, int dt, size_t i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// pair i of a rotated vector of `rot` dimensions: interleaved (2i, 2i+1) or half-split (i, i + rot/2)
__device__ __forceinline__ void pair_index(int i, int rot, int pairing, int& a, int& b) {
    if (pairing == 0) { a = 2 * i; b = 2 * i + 1; }
    else { a = i; b = i + rot / 2; }
}

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ src, int ld, int q_off, int kv_off, T* __restrict__ q_out,
                                      GfbPagedKV kv, GfbBatch b, const float* __restrict__ table, int table_len,
                                      const void* __restrict__ norm_w, int w_dt, float eps, int H, int d, int rot, int rank,
                                      int pairing, int append, int* status) {
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x;
    const int s = b.tok_seq[t];
    const int slot = b.slots[s];
    const int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    const T* row = src + (size_t)t * ld;
    const bool pos_ok = pos >= 0 && pos < table_len;
    if (!pos_ok && threadIdx.x == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
    const float* cs = table + (size_t)(pos_ok ? pos : 0) * rot;          // [rot/2][2]
    const int half = rot / 2;

    // every head's rotated query part
    const int qrow = rank + rot;
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, p = i - h * half;
        int ia, ib;
        pair_index(p, rot, pairing, ia, ib);
        const T* q = row + q_off + (size_t)h * (d + rot) + d;
        const float u = gfb_to_f32(q[ia]), v = gfb_to_f32(q[ib]);
        const float c = cs[2 * p], sn = cs[2 * p + 1];
        T* o = q_out + ((size_t)t * H + h) * qrow + rank;
        o[ia] = gfb_from_f32<T>(u * c - v * sn);
        o[ib] = gfb_from_f32<T>(v * c + u * sn);
    }
    if (!append) return;

    // the token's cache row: [normed latent | rotated shared key part]
    const int pi = pos / kv.page_size;
    int page = (pos_ok && pi < kv.max_pages) ? kv.page_table[(size_t)slot * kv.max_pages + pi] : -1;
    if (page < 0 || page >= kv.n_pages) {
        if (threadIdx.x == 0 && pos_ok) gfb_report(status, GFB_ERR_PAGE_TABLE, slot, pi);
        page = -1;
    }
    const T* dkv = row + kv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = gfb_to_f32(dkv[i]); ss += v * v; }
    ss = gfb_block_sum(ss, scratch);
    if (page < 0) return;
    const float r = 1.0f / sqrtf(ss / (float)rank + eps);
    T* krow = (T*)kv.k_pool + ((size_t)page * kv.page_size + (pos % kv.page_size)) * qrow;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        krow[i] = gfb_from_f32<T>(gfb_to_f32(dkv[i]) * r * ld_any(norm_w, w_dt, i));
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
        int ia, ib;
        pair_index(p, rot, pairing, ia, ib);
        const float u = gfb_to_f32(dkv[rank + ia]), v = gfb_to_f32(dkv[rank + ib]);
        const float c = cs[2 * p], sn = cs[2 * p + 1];
        krow[rank + ia] = gfb_from_f32<T>(u * c - v * sn);
        krow[rank + ib] = gfb_from_f32<T>(v * c + u * sn);
    }
}

// src [T, ld]: at q_off H heads of (d + rot) numbers (d unrotated, then rot rotated), at kv_off rank + rot numbers.
// q_out [T, H, rank + rot]: only the last rot numbers of every head are written here.  The cache entry has one
// key head of rank + rot numbers per token (its value pool is not used).  table float32 [table_len, rot/2, 2].
GFB_API int gfb_latent_prepare(const void* src, int dt, int ld, int q_off, int kv_off, void* q_out, void* k_pool,
                               const int* page_table, int max_pages, int page_size, int n_pages, const int* cu_seqlens,
                               const int* tok_seq, const int* slots, const int* lengths, int n_seqs, int n_tokens,
                               const float* table, int table_len, const void* norm_w, int w_dt, float eps, int H, int d,
                               int rot, int rank, int pairing, int append, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot % 2 || rot < 0 || rank <= 0) return gfb_fail("gfb_latent_prepare: rot = %d must be even, rank = %d positive", rot, rank);
    GfbPagedKV kv{k_pool, nullptr, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)src, ld, q_off,
                       kv_off, (__nv_bfloat16*)q_out, kv, b, table, table_len, norm_w, w_dt, eps, H, d, rot, rank, pairing, append, status);
    else if (dt == GFB_F32)
        e = gfb_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, (const float*)src, ld, q_off, kv_off,
                       (float*)q_out, kv, b, table, table_len, norm_w, w_dt, eps, H, d, rot, rank, pairing, append, status);
    else
        return gfb_fail("gfb_latent_prepare: unknown type %d", dt);
    return gfb_check(e, "gfb_latent_prepare");
}

// ---------------------------------------------------------------- a product with a weight per head -----
// out[t, h, n] = sum_k in[t, h, k] * W_h[k, n]  (kn = 1: W stored [H][K][N])  or  W_h[n, k]  (kn = 0: [H][N][K]),
// optionally times sigmoid(gate[t, h * N + n]).  A block takes TT tokens of one head; the inputs sit in shared
// memory as 32-bit numbers; a thread owns output columns and adds over k in ascending order.
constexpr int HL_TT = 8;
constexpr int HL_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(HL_THREADS)
headwise_linear_kernel(const T* __restrict__ in, int ld_in, int in_off, int in_stride, const T* __restrict__ w, int kn,
                       T* __restrict__ out, int ld_out, int out_off, int out_stride, const T* __restrict__ gate, int ld_gate,
                       int gate_off, int n_tokens, int K, int N) {
    extern __shared__ float xs[];                 // [HL_TT][K]
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int h = blockIdx.y;
    const int t0 = blockIdx.x * HL_TT;
    const int nt = min(HL_TT, n_tokens - t0);
    for (int i = threadIdx.x; i < HL_TT * K; i += blockDim.x) {
        const int tt = i / K, k = i - tt * K;
        xs[i] = tt < nt ? gfb_to_f32(in[(size_t)(t0 + tt) * ld_in + in_off + (size_t)h * in_stride + k]) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (size_t)h * K * N;
    if (kn) {
        for (int n = threadIdx.x; n < N; n += blockDim.x) {
            float acc[HL_TT];
#pragma unroll
            for (int tt = 0; tt < HL_TT; tt++) acc[tt] = 0.f;
            for (int k = 0; k < K; k++) {
                const float wv = gfb_to_f32(wh[(size_t)k * N + n]);
#pragma unroll
                for (int tt = 0; tt < HL_TT; tt++) acc[tt] = fmaf(xs[tt * K + k], wv, acc[tt]);
            }
#pragma unroll
            for (int tt = 0; tt < HL_TT; tt++)
                if (tt < nt) {
                    float v = acc[tt];
                    if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gfb_to_f32(gate[(size_t)(t0 + tt) * ld_gate + gate_off + (size_t)h * N + n])));
                    out[(size_t)(t0 + tt) * ld_out + out_off + (size_t)h * out_stride + n] = gfb_from_f32<T>(v);
                }
        }
    } else {
        // a warp per output column: lanes stride over k, then a fixed tree adds the 32 partial sums
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        for (int n = warp; n < N; n += nwarp) {
            float acc[HL_TT];
#pragma unroll
            for (int tt = 0; tt < HL_TT; tt++) acc[tt] = 0.f;
            for (int k = lane; k < K; k += 32) {
                const float wv = gfb_to_f32(wh[(size_t)n * K + k]);
#pragma unroll
                for (int tt = 0; tt < HL_TT; tt++) acc[tt] = fmaf(xs[tt * K + k], wv, acc[tt]);
            }
#pragma unroll
            for (int tt = 0; tt < HL_TT; tt++) acc[tt] = gfb_warp_sum(acc[tt]);
            if (lane == 0) {
#pragma unroll
                for (int tt = 0; tt < HL_TT; tt++)
                    if (tt < nt) {
                        float v = acc[tt];
                        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gfb_to_f32(gate[(size_t)(t0 + tt) * ld_gate + gate_off + (size_t)h * N + n])));
                        out[(size_t)(t0 + tt) * ld_out + out_off + (size_t)h * out_stride + n] = gfb_from_f32<T>(v);
                    }
            }
        }
    }
}

// in [T, ld_in]: head h's K inputs start at column in_off + h * in_stride; out [T, ld_out] likewise; w [H, K, N] (kn)
// or [H, N, K]; gate (or null) [T, ld_gate] with head h's N gate values at column gate_off + h * N.  One type for all.
GFB_API int gfb_headwise_linear(const void* in, int dt, int ld_in, int in_off, int in_stride, const void* w, int kn, void* out,
                                int ld_out, int out_off, int out_stride, const void* gate, int ld_gate, int gate_off,
                                int n_tokens, int H, int K, int N, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || N <= 0) return 0;
    if (K <= 0) return gfb_fail("gfb_headwise_linear: K = %d", K);
    if (H > 65535) return gfb_fail("gfb_headwise_linear: %d heads exceed the grid limit", H);
    const size_t smem = (size_t)HL_TT * K * sizeof(float);
    if (smem > 160 * 1024) return gfb_fail("gfb_headwise_linear: K = %d does not fit shared memory", K);
    dim3 grid((n_tokens + HL_TT - 1) / HL_TT, H);
    cudaError_t e;
#define GO(T)                                                                                                               \
    do {                                                                                                                    \
        static size_t allowed = 48 * 1024;                                                                                  \
        if (smem > allowed) {                                                                                               \
            cudaFuncSetAttribute(headwise_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);       \
            allowed = 160 * 1024;                                                                                           \
        }                                                                                                                   \
        e = gfb_launch(headwise_linear_kernel<T>, grid, dim3(HL_THREADS), smem, stream, (const T*)in, ld_in, in_off, in_stride, \
                       (const T*)w, kn, (T*)out, ld_out, out_off, out_stride, (const T*)gate, ld_gate, gate_off, n_tokens, K, N); \
    } while (0)
    if (dt == GFB_BF16) GO(__nv_bfloat16);
    else if (dt == GFB_F32) GO(float);
    else return gfb_fail("gfb_headwise_linear: unknown type %d", dt);
#undef GO
    return gfb_check(e, "gfb_headwise_linear");
}
