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
// gfb_headwise_linear  out[t, h, :] = in[t, h, :] W_h with a weight per head (the two expansions above), strided
//                      inputs and outputs, optionally times sigmoid(gate[t, h, :]).
// gfb_latent_attention attention on the cached rows for bfloat16 on tensor cores (below).
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

// ---------------------------------------------------------------- a product with a weight per head, on tensor cores -----
// out[t, h, n] = sum_k in[t, h, k] * W_h[k, n] (see below) for bfloat16 with 16-byte aligned rows, `mma.sync.m16n8k16`: a block takes 64 tokens (four warps of 16 rows) of one head and 64 output columns and
// walks over k in pieces of 64; the weight piece [k][n] is the B operand, transposed on its way into the registers.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem));
}
// a barrier of the two warps that share 16 query rows (named barriers 1..4; 0 is the block's)
__device__ __forceinline__ void pair_barrier(int pair) { asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int HT_ROWS = 64, HT_COLS = 64, HT_K = 64, HT_PAD = 8;

__global__ void __launch_bounds__(128)
headwise_linear_tc_kernel(const __nv_bfloat16* __restrict__ in, int ld_in, int in_off, int in_stride, const __nv_bfloat16* __restrict__ w,
                          __nv_bfloat16* __restrict__ out, int ld_out, int out_off, int out_stride, const __nv_bfloat16* __restrict__ gate,
                          int ld_gate, int gate_off, int n_tokens, int K, int N) {
    __shared__ __align__(16) __nv_bfloat16 sA[HT_ROWS][HT_K + HT_PAD];
    __shared__ __align__(16) __nv_bfloat16 sW[HT_K][HT_COLS + HT_PAD];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.x * HT_ROWS, n0 = blockIdx.z * HT_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* a_base = in + in_off + (size_t)h * in_stride;
    const __nv_bfloat16* w_base = w + (size_t)h * K * N;
    float acc[HT_COLS / 8][4];
#pragma unroll
    for (int j = 0; j < HT_COLS / 8; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HT_K) {
        __syncthreads();
        for (int c = tid; c < HT_ROWS * (HT_K / 8); c += 128) {              // 16-byte pieces; K and N are multiples of 8
            const int r = c / (HT_K / 8), cc = (c % (HT_K / 8)) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t0 + r < n_tokens && k0 + cc < K) v = *reinterpret_cast<const uint4*>(a_base + (size_t)(t0 + r) * ld_in + k0 + cc);
            *reinterpret_cast<uint4*>(&sA[r][cc]) = v;
        }
        for (int c = tid; c < HT_K * (HT_COLS / 8); c += 128) {
            const int r = c / (HT_COLS / 8), cc = (c % (HT_COLS / 8)) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (k0 + r < K && n0 + cc < N) v = *reinterpret_cast<const uint4*>(w_base + (size_t)(k0 + r) * N + n0 + cc);
            *reinterpret_cast<uint4*>(&sW[r][cc]) = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HT_K; kk += 16) {
            uint32_t a[4];
            ldsm_x4(a, &sA[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][kk + 8 * (lane >> 4)]);
#pragma unroll
            for (int j = 0; j < HT_COLS / 8; j += 2) {
                uint32_t bb[4];
                ldsm_x4_trans(bb, &sW[kk + (lane & 7) + 8 * ((lane >> 3) & 1)][(j + (lane >> 4)) * 8]);
                mma_bf16(acc[j], a, bb[0], bb[1]);
                mma_bf16(acc[j + 1], a, bb[2], bb[3]);
            }
        }
    }
    const int r0 = t0 + warp * 16 + (lane >> 2);
#pragma unroll
    for (int j = 0; j < HT_COLS / 8; j++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int t = r0 + 8 * (e >> 1), n = n0 + j * 8 + 2 * (lane & 3) + (e & 1);
            if (t < n_tokens && n < N) {
                float v = acc[j][e];
                if (gate != nullptr) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * ld_gate + gate_off + (size_t)h * N + n])));
                out[(size_t)t * ld_out + out_off + (size_t)h * out_stride + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

// ---------------------------------------------------------------- a product with a weight per head -----
// out[t, h, n] = sum_k in[t, h, k] * W_h[k, n]  (W stored [H][K][N]), optionally times sigmoid(gate[t, h * N + n]).
// A block takes HL_TT tokens of one head and 128 output columns; its inputs sit in shared memory as 32-bit numbers.
// Thread (column, slice) adds every HL_KS-th k in ascending order (the weight loads of a warp are one row piece,
// coalesced); the slices' sums are then added in ascending order through shared memory.
constexpr int HL_TT = 8;
constexpr int HL_COLS = 128;
constexpr int HL_KS = 4;
constexpr int HL_THREADS = HL_COLS * HL_KS;

template <typename T>
__global__ void __launch_bounds__(HL_THREADS)
headwise_linear_kernel(const T* __restrict__ in, int ld_in, int in_off, int in_stride, const T* __restrict__ w,
                       T* __restrict__ out, int ld_out, int out_off, int out_stride, const T* __restrict__ gate, int ld_gate,
                       int gate_off, int n_tokens, int K, int N) {
    extern __shared__ float xs[];                 // [HL_TT][K], then [HL_KS][HL_TT][HL_COLS] partial sums
    float* part = xs + (size_t)HL_TT * K;
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
    const int c = threadIdx.x % HL_COLS, ks = threadIdx.x / HL_COLS;
    const int n = blockIdx.z * HL_COLS + c;
    const T* wh = w + (size_t)h * K * N;
    float acc[HL_TT];
#pragma unroll
    for (int tt = 0; tt < HL_TT; tt++) acc[tt] = 0.f;
    if (n < N) {
#pragma unroll 4
        for (int k = ks; k < K; k += HL_KS) {
            const float wv = gfb_to_f32(wh[(size_t)k * N + n]);
#pragma unroll
            for (int tt = 0; tt < HL_TT; tt++) acc[tt] = fmaf(xs[tt * K + k], wv, acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < HL_TT; tt++) part[((size_t)ks * HL_TT + tt) * HL_COLS + c] = acc[tt];
    __syncthreads();
    for (int i = threadIdx.x; i < HL_TT * HL_COLS; i += blockDim.x) {
        const int tt = i / HL_COLS, cc = i - tt * HL_COLS, col = blockIdx.z * HL_COLS + cc;
        if (tt >= nt || col >= N) continue;
        float v = part[(size_t)tt * HL_COLS + cc];
#pragma unroll
        for (int s = 1; s < HL_KS; s++) v += part[((size_t)s * HL_TT + tt) * HL_COLS + cc];
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gfb_to_f32(gate[(size_t)(t0 + tt) * ld_gate + gate_off + (size_t)h * N + col])));
        out[(size_t)(t0 + tt) * ld_out + out_off + (size_t)h * out_stride + col] = gfb_from_f32<T>(v);
    }
}

// in [T, ld_in]: head h's K inputs start at column in_off + h * in_stride; out [T, ld_out] likewise; w [H, K, N]; gate (or
// null) [T, ld_gate] with head h's N gate values at column gate_off + h * N.  One type for all.
GFB_API int gfb_headwise_linear(const void* in, int dt, int ld_in, int in_off, int in_stride, const void* w, void* out,
                                int ld_out, int out_off, int out_stride, const void* gate, int ld_gate, int gate_off,
                                int n_tokens, int H, int K, int N, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || N <= 0) return 0;
    if (K <= 0) return gfb_fail("gfb_headwise_linear: K = %d", K);
    if (H > 65535 || (N + HL_COLS - 1) / HL_COLS > 65535) return gfb_fail("gfb_headwise_linear: %d heads of %d columns exceed the grid limit", H, N);
    if (dt == GFB_BF16 && K % 16 == 0 && N % 8 == 0 && ld_in % 8 == 0 && in_off % 8 == 0 && in_stride % 8 == 0 &&
        (((uintptr_t)in | (uintptr_t)w) & 15) == 0) {
        dim3 grid((n_tokens + HT_ROWS - 1) / HT_ROWS, H, (N + HT_COLS - 1) / HT_COLS);
        cudaError_t e = gfb_launch(headwise_linear_tc_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)in, ld_in, in_off, in_stride,
                                   (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ld_out, out_off, out_stride, (const __nv_bfloat16*)gate,
                                   ld_gate, gate_off, n_tokens, K, N);
        return gfb_check(e, "gfb_headwise_linear (tensor cores)");
    }
    const size_t smem = ((size_t)HL_TT * K + (size_t)HL_KS * HL_TT * HL_COLS) * sizeof(float);
    if (smem > 160 * 1024) return gfb_fail("gfb_headwise_linear: K = %d does not fit shared memory", K);
    dim3 grid((n_tokens + HL_TT - 1) / HL_TT, H, (N + HL_COLS - 1) / HL_COLS);
    cudaError_t e;
#define GO(T)                                                                                                               \
    do {                                                                                                                    \
        static size_t allowed = 48 * 1024;                                                                                  \
        if (smem > allowed) {                                                                                               \
            cudaFuncSetAttribute(headwise_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);       \
            allowed = 160 * 1024;                                                                                           \
        }                                                                                                                   \
        e = gfb_launch(headwise_linear_kernel<T>, grid, dim3(HL_THREADS), smem, stream, (const T*)in, ld_in, in_off, in_stride, \
                       (const T*)w, (T*)out, ld_out, out_off, out_stride, (const T*)gate, ld_gate, gate_off, n_tokens, K, N); \
    } while (0)
    if (dt == GFB_BF16) GO(__nv_bfloat16);
    else if (dt == GFB_F32) GO(float);
    else return gfb_fail("gfb_headwise_linear: unknown type %d", dt);
#undef GO
    return gfb_check(e, "gfb_headwise_linear");
}

// ---------------------------------------------------------------- attention on the latent, many queries ----
// All heads read the same cached rows: keys are the whole rows (Dk = rank + rot numbers), values their first `rank`
// numbers.  So the rows of one MMA are (token, head) pairs of ONE sequence, 64 of them per block (four warps of 16),
// and a tile of 32 cached rows, fetched once into shared memory (cp.async, two stages), serves as the B operand of
// S = Q K^T (as stored) and of O += P V (transposed on the way into the registers).  Two warps share 16 query rows:
// each scores half of the tile's keys, they agree on the rows' maxima and exchange their softmax weights through shared
// memory (two barriers of 64 threads per tile), and each keeps half of the value columns of O in registers (128 numbers
// per thread at rank 512).  bfloat16 operands on `mma.sync.m16n8k16`, scores, softmax and sums in 32-bit; the softmax
// weights are rounded to bfloat16 for the second product.  Keys are masked per row by the row's own position.
constexpr int LA_ROWS = 64;           // query rows per block
constexpr int LA_KEYS = 32;           // cached rows per tile
constexpr int LA_THREADS = 256;
constexpr int LA_PAD = 8;             // bfloat16 numbers of padding per shared-memory row: ldmatrix rows fall into distinct banks

// NT: value n-tiles (of 8 columns) a warp may hold: rank / 2 <= 8 * NT
template <int NT>
__global__ void __launch_bounds__(LA_THREADS, 1)
latent_attention_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, GfbPagedKV kv, GfbBatch b,
                        int H, int Dk, int R, float scale_log2, int n_splits, float* __restrict__ partial, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DkP = Dk + LA_PAD;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [LA_ROWS][DkP]
    __nv_bfloat16* sK = sQ + (size_t)LA_ROWS * DkP;                             // [2][LA_KEYS][DkP]
    __shared__ __align__(16) __nv_bfloat16 sP[4][16][LA_KEYS + LA_PAD];         // a warp pair's softmax weights of the tile
    __shared__ float sMax[4][2][16], sSum[4][2][16];                            // each half's row maxima of the tile; row sums at the end
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x;
    const int t0 = b.cu_seqlens[s], n_rows = (b.cu_seqlens[s + 1] - t0) * H;
    // the latest rows see the most keys: they come first, so that the blocks of the last round are the short ones
    const int m0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * LA_ROWS;
    if (m0 >= n_rows) return;
    const int slot = b.slots[s], start = b.lengths[slot];
    const int rows_here = min(LA_ROWS, n_rows - m0);
    const int last_pos = start + (m0 + rows_here - 1) / H;                      // the latest position any row of the block sees
    const int all_tiles = last_pos / LA_KEYS + 1;
    // with n_splits > 1 (a decode step) the block takes one slice of the cached rows and leaves its unnormalised sums
    const int per_split = (all_tiles + n_splits - 1) / n_splits;
    const int tile_lo = blockIdx.z * per_split, n_tiles = min(all_tiles, tile_lo + per_split);
    const int* pt = kv.page_table + (size_t)slot * kv.max_pages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunks = Dk / 8;                                                  // 16-byte pieces of a row

    auto load_keys = [&](int stage, int tile) {
        const int key0 = tile * LA_KEYS;
        const int pi = key0 / kv.page_size;
        int page = pi < kv.max_pages ? pt[pi] : -1;
        if (page < 0 || page >= kv.n_pages) {
            if (tid == 0) gfb_report(status, GFB_ERR_PAGE_TABLE, slot, pi);
            page = 0;
        }
        const __nv_bfloat16* src = (const __nv_bfloat16*)kv.k_pool + ((size_t)page * kv.page_size + key0 % kv.page_size) * Dk;
        __nv_bfloat16* dst = sK + (size_t)stage * LA_KEYS * DkP;
        for (int c = tid; c < LA_KEYS * chunks; c += LA_THREADS) {
            const int r = c / chunks, cc = c - r * chunks;
            cp_async16(dst + (size_t)r * DkP + cc * 8, src + (size_t)r * Dk + cc * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (tile_lo < n_tiles) load_keys(tile_lo & 1, tile_lo);
    // the block's query rows (rows beyond the sequence's are zero)
    const __nv_bfloat16* qsrc = q + ((size_t)t0 * H + m0) * Dk;
    for (int c = tid; c < LA_ROWS * chunks; c += LA_THREADS) {
        const int r = c / chunks, cc = c - r * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_here) v = *reinterpret_cast<const uint4*>(qsrc + (size_t)r * Dk + cc * 8);
        *reinterpret_cast<uint4*>(sQ + (size_t)r * DkP + cc * 8) = v;
    }

    const int pair = warp & 3, rw = pair * 16;         // the warp's 16 query rows, shared with the warp `pair + 4`
    const int half = warp >> 2;                        // which half of a tile's keys it scores and of the value columns it keeps
    const int nt_all = R / 8, nt_lo = half == 0 ? 0 : (nt_all + 1) / 2, nt_n = half == 0 ? (nt_all + 1) / 2 : nt_all - (nt_all + 1) / 2;
    const int r0 = rw + (lane >> 2);                   // rows of this thread's accumulator values: r0 and r0 + 8
    const int pos0 = (r0 < rows_here) ? start + (m0 + r0) / H : -1, pos1 = (r0 + 8 < rows_here) ? start + (m0 + r0 + 8) / H : -1;
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    if (tile_lo >= n_tiles) __syncthreads();            // (an empty slice still leaves its neutral sums below)
    for (int tile = tile_lo; tile < n_tiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < n_tiles) {
            load_keys(stage ^ 1, tile + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* kt = sK + (size_t)stage * LA_KEYS * DkP;
        // scores of 16 rows x 16 keys: the two warps of a pair take half of the tile's keys each
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
        for (int kk = 0; kk < Dk; kk += 16) {
            uint32_t a[4], bb[4];
            ldsm_x4(a, sQ + (size_t)(rw + (lane & 7) + 8 * ((lane >> 3) & 1)) * DkP + kk + 8 * (lane >> 4));
            ldsm_x4(bb, kt + (size_t)((2 * half + (lane >> 4)) * 8 + (lane & 7)) * DkP + kk + 8 * ((lane >> 3) & 1));
            mma_bf16(sc[0], a, bb[0], bb[1]);
            mma_bf16(sc[1], a, bb[2], bb[3]);
        }
        // mask by each row's position; the pair agrees on the rows' maxima through shared memory
        const int key0 = tile * LA_KEYS + 16 * half + 2 * (lane & 3);
        float t0m = -INFINITY, t1m = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int key = key0 + j * 8 + e;
                sc[j][e] = key <= pos0 ? sc[j][e] * scale_log2 : -INFINITY;
                sc[j][2 + e] = key <= pos1 ? sc[j][2 + e] * scale_log2 : -INFINITY;
                t0m = fmaxf(t0m, sc[j][e]);
                t1m = fmaxf(t1m, sc[j][2 + e]);
            }
        }
        t0m = fmaxf(t0m, __shfl_xor_sync(0xffffffffu, t0m, 1));
        t0m = fmaxf(t0m, __shfl_xor_sync(0xffffffffu, t0m, 2));
        t1m = fmaxf(t1m, __shfl_xor_sync(0xffffffffu, t1m, 1));
        t1m = fmaxf(t1m, __shfl_xor_sync(0xffffffffu, t1m, 2));
        if ((lane & 3) == 0) { sMax[pair][half][lane >> 2] = t0m; sMax[pair][half][(lane >> 2) + 8] = t1m; }
        pair_barrier(pair);
        t0m = fmaxf(t0m, sMax[pair][half ^ 1][lane >> 2]);
        t1m = fmaxf(t1m, sMax[pair][half ^ 1][(lane >> 2) + 8]);
        const float n0 = fmaxf(mx0, t0m), n1 = fmaxf(mx1, t1m);
        const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;       // a row that sees nothing yet
        const float al0 = exp2f(mx0 - u0), al1 = exp2f(mx1 - u1);                             // exp2(-inf) = 0
        mx0 = n0;
        mx1 = n1;
        float s0 = 0.f, s1 = 0.f;                       // sums over this warp's keys only; the halves are added at the end
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float p00 = exp2f(sc[j][0] - u0), p01 = exp2f(sc[j][1] - u0), p10 = exp2f(sc[j][2] - u1), p11 = exp2f(sc[j][3] - u1);
            s0 += p00 + p01;
            s1 += p10 + p11;
            const int col = 16 * half + 8 * j + 2 * (lane & 3);
            *reinterpret_cast<uint32_t*>(&sP[pair][lane >> 2][col]) = pack_bf16(p00, p01);
            *reinterpret_cast<uint32_t*>(&sP[pair][(lane >> 2) + 8][col]) = pack_bf16(p10, p11);
        }
        pair_barrier(pair);
        uint32_t pa[LA_KEYS / 16][4];
#pragma unroll
        for (int kb = 0; kb < LA_KEYS / 16; kb++) ldsm_x4(pa[kb], &sP[pair][(lane & 7) + 8 * ((lane >> 3) & 1)][kb * 16 + 8 * (lane >> 4)]);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        l0 = l0 * al0 + s0;
        l1 = l1 * al1 + s1;
        // O = O * alpha + P V over the warp's value columns
#pragma unroll
        for (int j = 0; j < NT; j++) {
            o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1;
        }
#pragma unroll
        for (int kb = 0; kb < LA_KEYS / 16; kb++) {
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                if (j < nt_n) {
                    // the second tile of the pair may lie beyond the warp's columns (an odd count): it reads the next
                    // columns of the row, which exist (Dk > R), and its result is dropped
                    uint32_t vb[4];
                    ldsm_x4_trans(vb, kt + (size_t)(kb * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * DkP + (nt_lo + j + (lane >> 4)) * 8);
                    mma_bf16(o[j], pa[kb], vb[0], vb[1]);
                    if (j + 1 < NT) mma_bf16(o[j + 1], pa[kb], vb[2], vb[3]);
                }
            }
        }
        __syncthreads();                               // the stage is free for the tile after next
    }
    // the row sums of the two halves (both under the same maxima)
    if ((lane & 3) == 0) { sSum[pair][half][lane >> 2] = l0; sSum[pair][half][(lane >> 2) + 8] = l1; }
    pair_barrier(pair);
    l0 += sSum[pair][half ^ 1][lane >> 2];
    l1 += sSum[pair][half ^ 1][(lane >> 2) + 8];
    if (n_splits > 1) {
        // [row][split][R values, maximum (base-2 exponent), sum]
        float* base = partial + (((size_t)t0 * H + m0) * n_splits + blockIdx.z) * (R + 2);
        const size_t row_stride = (size_t)n_splits * (R + 2);
#pragma unroll
        for (int j = 0; j < NT; j++) {
            if (j < nt_n) {
                const int col = (nt_lo + j) * 8 + 2 * (lane & 3);
                if (r0 < rows_here) *reinterpret_cast<float2*>(base + (size_t)r0 * row_stride + col) = make_float2(o[j][0], o[j][1]);
                if (r0 + 8 < rows_here) *reinterpret_cast<float2*>(base + (size_t)(r0 + 8) * row_stride + col) = make_float2(o[j][2], o[j][3]);
            }
        }
        if (half == 0 && (lane & 3) == 0) {
            if (r0 < rows_here) { base[(size_t)r0 * row_stride + R] = mx0; base[(size_t)r0 * row_stride + R + 1] = l0; }
            if (r0 + 8 < rows_here) { base[(size_t)(r0 + 8) * row_stride + R] = mx1; base[(size_t)(r0 + 8) * row_stride + R + 1] = l1; }
        }
        return;
    }
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    __nv_bfloat16* orow = out + ((size_t)t0 * H + m0) * R;
#pragma unroll
    for (int j = 0; j < NT; j++) {
        if (j < nt_n) {
            const int col = (nt_lo + j) * 8 + 2 * (lane & 3);
            if (r0 < rows_here) *reinterpret_cast<uint32_t*>(orow + (size_t)r0 * R + col) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
            if (r0 + 8 < rows_here) *reinterpret_cast<uint32_t*>(orow + (size_t)(r0 + 8) * R + col) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
        }
    }
}

// The slices of a row: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M the largest m_s, slices in ascending order.
__global__ void latent_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int n_splits, int R) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const size_t row = blockIdx.x;
    const float* base = partial + row * n_splits * (R + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, base[(size_t)s * (R + 2) + R]);
    float l = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float m = base[(size_t)s * (R + 2) + R];
        if (m != -INFINITY) l += base[(size_t)s * (R + 2) + R + 1] * exp2f(m - M);
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float m = base[(size_t)s * (R + 2) + R];
            if (m != -INFINITY) v += base[(size_t)s * (R + 2) + c] * exp2f(m - M);
        }
        out[row * R + c] = __float2bfloat16_rn(v * inv);
    }
}

// q bfloat16 [T, H, Dk] (Dk = rank + rot), out bfloat16 [T, H * rank]; the cache entry holds one row of Dk numbers per
// token in pages of a multiple of 32 tokens.  Needs Dk % 16 == 0, rank % 16 == 0, rank <= 512, rank < Dk.  n_splits > 1:
// every sequence's cached rows are cut into that many slices with a block each, whose sums go through `partial`
// (float32 [T * H, n_splits, rank + 2]) and a second kernel.
GFB_API int gfb_latent_attention(const void* q, void* out, void* k_pool, const int* page_table, int max_pages, int page_size,
                                 int n_pages, const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                                 int n_seqs, int n_tokens, int max_q_len, int H, int Dk, int R, float scale, int n_splits,
                                 float* partial, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Dk % 16 || R % 16 || R > 512 || R >= Dk || page_size % LA_KEYS)
        return gfb_fail("gfb_latent_attention: rows of %d with %d value columns in pages of %d do not fit the kernel", Dk, R, page_size);
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pool) & 15) != 0) return gfb_fail("gfb_latent_attention: operands must be 16-byte aligned");
    GfbPagedKV kv{k_pool, nullptr, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const size_t smem = (size_t)(LA_ROWS + 2 * LA_KEYS) * (Dk + LA_PAD) * sizeof(__nv_bfloat16);
    if (smem > 220 * 1024) return gfb_fail("gfb_latent_attention: rows of %d numbers do not fit shared memory", Dk);
    const long tiles = ((long)max_q_len * H + LA_ROWS - 1) / LA_ROWS;
    if (tiles > 65535) return gfb_fail("gfb_latent_attention: %ld row tiles exceed the grid limit", tiles);
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 1 && partial == nullptr) return gfb_fail("gfb_latent_attention: slices need room for their sums");
    dim3 grid(n_seqs, (unsigned)tiles, n_splits);
    const float scale_log2 = scale * 1.4426950408889634f;
    const int nt = (R / 8 + 1) / 2;
    cudaError_t e;
#define GO(NT)                                                                                                              \
    do {                                                                                                                    \
        e = cudaFuncSetAttribute(latent_attention_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        if (e != cudaSuccess) return gfb_fail("gfb_latent_attention: %s", cudaGetErrorString(e));                           \
        e = gfb_launch(latent_attention_kernel<NT>, grid, dim3(LA_THREADS), smem, stream, (const __nv_bfloat16*)q,          \
                       (__nv_bfloat16*)out, kv, b, H, Dk, R, scale_log2, n_splits, partial, status);                        \
    } while (0)
    if (nt <= 8) GO(8);
    else if (nt <= 16) GO(16);
    else GO(32);
#undef GO
    if (gfb_check(e, "gfb_latent_attention")) return 1;
    if (n_splits == 1) return 0;
    e = gfb_launch(latent_combine_kernel, dim3((unsigned)n_tokens * H), dim3(128), 0, stream, (const float*)partial, (__nv_bfloat16*)out,
                   n_splits, R);
    return gfb_check(e, "gfb_latent_attention (combine)");
}
