// Layer norm with weight and bias over the 32-bit residual stream, and the "normed branch" sum of
// sandwich blocks:
//
//     LN(v; w, b) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w + b
//
// One kernel does, per row, up to two things in one pass:
//   (1) branch sum:  x[row] += mult * LN(y[row]; pw, pb)     (y: a sublayer's 32-bit output, or the
//       partial sums [S][T][D] of a product that was split over K, added here in ascending order)
//   (2) norm:        out[r] = LN(x[row]; w, b)                (in the compute type)
// so that the norm behind a sublayer and the norm ahead of the next one cost one trip over the row.
// Means and variances are 32-bit; the variance is the mean of the squared deviations (two passes
// over the row, which sits in shared memory).  `rms` = 1 selects the root-mean-square form (no
// mean, no bias) with the same interface.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float ld_w(const void* p, int dt, int i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// statistics of the row held in `row` (shared memory): returns (mean, 1/sqrt(var + eps)); rms: (0, 1/sqrt(mean sq + eps))
__device__ __forceinline__ float2 row_stats(const float* row, int D, float eps, int rms, float* scratch) {
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) s += row[i];
        mean = gfb_block_sum(s, scratch) / (float)D;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { float dv = row[i] - mean; ss += dv * dv; }
    ss = gfb_block_sum(ss, scratch);
    return make_float2(mean, 1.0f / sqrtf(ss / (float)D + eps));
}

template <typename TO>
__global__ void layernorm_kernel(float* __restrict__ x, const float* __restrict__ y, int S, size_t slice,
                                 const void* pw, const void* pb, int p_dt, float peps, float mult,
                                 const void* w, const void* b, int w_dt, float eps, TO* __restrict__ out,
                                 const int* __restrict__ rows, int D, int rms) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int r = blockIdx.x;
    const size_t base = (size_t)(rows ? rows[r] : r) * D;
    if (y != nullptr) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = y[base + i];
            for (int k = 1; k < S; k++) v += y[(size_t)k * slice + base + i];
            row[i] = v;
        }
        __syncthreads();
        const float2 st = row_stats(row, D, peps, rms, scratch);
        __syncthreads();
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float n = (row[i] - st.x) * st.y * ld_w(pw, p_dt, i);
            if (!rms) n += ld_w(pb, p_dt, i);
            const float v = x[base + i] + mult * n;
            x[base + i] = v;
            row[i] = v;
        }
    } else if (out != nullptr) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) row[i] = x[base + i];
    }
    if (out == nullptr) return;
    __syncthreads();
    const float2 st = row_stats(row, D, eps, rms, scratch);
    TO* o = out + (size_t)r * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float n = (row[i] - st.x) * st.y * ld_w(w, w_dt, i);
        if (!rms) n += ld_w(b, w_dt, i);
        o[i] = gfb_from_f32<TO>(n);
    }
}

// x float32 [T, D].  y (or null): float32 [max(S,1)][T][D] (S = 0 or 1: one tensor; S > 1: partial sums), with its norm
// (pw, pb, p_dt, peps) and the factor mult.  out (or null): [R, D] of type out_dt with its norm (w, b, w_dt, eps);
// rows (or null) gathers input rows for `out` and cannot be combined with y.
GFB_API int gfb_layernorm(float* x, const float* y, int S, long slice, const void* pw, const void* pb, int p_dt, float peps,
                          float mult, const void* w, const void* b, int w_dt, float eps, void* out, int out_dt,
                          const int* rows, int R, int D, int rms, cudaStream_t stream) {
    if (R <= 0 || D <= 0) return 0;
    if (y != nullptr && rows != nullptr) return gfb_fail("gfb_layernorm: a branch sum cannot be combined with a row gather");
    if (y == nullptr && out == nullptr) return 0;
    if ((size_t)D * sizeof(float) > 200 * 1024) return gfb_fail("gfb_layernorm: a row of %d elements does not fit shared memory", D);
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    const size_t smem = (size_t)D * sizeof(float);
    cudaError_t e;
#define GO(TO)                                                                                                         \
    do {                                                                                                               \
        static size_t allowed = 48 * 1024;                                                                             \
        if (smem > allowed) {                                                                                          \
            cudaFuncSetAttribute(layernorm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);       \
            allowed = 200 * 1024;                                                                                      \
        }                                                                                                              \
        e = gfb_launch(layernorm_kernel<TO>, dim3(R), dim3(threads), smem, stream, x, y, S, (size_t)slice, pw, pb, p_dt, peps, \
                       mult, w, b, w_dt, eps, (TO*)out, rows, D, rms);                                                 \
    } while (0)
    if (out == nullptr || out_dt == GFB_F32) GO(float);
    else if (out_dt == GFB_BF16) GO(__nv_bfloat16);
    else return gfb_fail("gfb_layernorm: unknown output type %d", out_dt);
#undef GO
    return gfb_check(e, "gfb_layernorm");
}
