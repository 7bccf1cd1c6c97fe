// Row-wise kernels around the residual stream that arrangements other than the pre-norm block
// need: an absolute sinusoidal position vector added to the embedded tokens, the add of two
// sublayers' outputs at once (a block whose mixer and feed-forward read the same norm), a
// gated look-up of a per-token table, and the add of a normalised product.
//
// A product reaches these kernels as float32 slices [S, T, N] that are summed in ascending s, as
// everywhere in the library; all sums and norms are float32.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// x[t, 2i] += sin(pos[t] * f[i]), x[t, 2i + 1] += cos(pos[t] * f[i]); angles in float32
// ------------------------------------------------------------------------------------------
__global__ void add_sinusoid_kernel(float *__restrict__ x, const int *__restrict__ positions,
                                    const float *__restrict__ freq, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    float *row = x + (size_t)t * d;
    for (int i = threadIdx.x; 2 * i < d; i += blockDim.x) {
        float s, c;
        sincosf(p * freq[i], &s, &c);
        row[2 * i] += s;
        if (2 * i + 1 < d) row[2 * i + 1] += c;
    }
}

KESTREL_API int kestrel_add_sinusoid(float *x, const int *positions, const float *freq, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0, "add_sinusoid: bad sizes T=%d d=%d", T, d);
    kestrel_launch(add_sinusoid_kernel, dim3(T), dim3(128), 0, stream, x, positions, freq, d);
    return kestrel_check_launch("add_sinusoid");
}

// ------------------------------------------------------------------------------------------
// residual[t] += sum_s a[s, t] + sum_s b[s, t]  (b may be null); cast[t] = residual[t] in the
// storage type (cast may be null).  The order of the sum is fixed: a's slices, then b's.
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void add_two_kernel(float *__restrict__ residual, const float *__restrict__ a, int Sa, size_t stride_a,
                               const float *__restrict__ b, int Sb, size_t stride_b, TOut *__restrict__ cast, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float va = sum_slices(a, Sa, stride_a, idx), vb = Sb > 0 ? sum_slices(b, Sb, stride_b, idx) : 0.f;
    float v = residual[idx] + (va + vb);
    residual[idx] = v;
    if (cast) cast[idx] = from_f32<TOut>(v);
}

KESTREL_API int kestrel_add_two(float *residual, const float *a, int Sa, long long stride_a, const float *b, int Sb, long long stride_b,
                                void *cast, int cast_dtype, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && a && Sa > 0 && (b || Sb == 0), "add_two: bad arguments");
    size_t n = (size_t)T * d;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (cast_dtype == KESTREL_F32)
        kestrel_launch(add_two_kernel<float>, dim3(blocks), dim3(256), 0, stream, residual, a, Sa, (size_t)stride_a, b, Sb, (size_t)stride_b, (float *)cast, n);
    else if (cast_dtype == KESTREL_BF16)
        kestrel_launch(add_two_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, residual, a, Sa, (size_t)stride_a, b, Sb, (size_t)stride_b, (__nv_bfloat16 *)cast, n);
    else
        return kestrel_fail(-2, "add_two: unknown dtype %d", cast_dtype);
    return kestrel_check_launch("add_two");
}

// ------------------------------------------------------------------------------------------
// out[t, i] = gelu_tanh(sum_s g[s, t, i]) * table[ids[t], col0 + i], i < n
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TW, typename TOut>
__global__ void gelu_table_mul_kernel(const float *__restrict__ g, int S, size_t slice_stride, int ld, const TW *__restrict__ table,
                                      int table_ld, int col0, const int *__restrict__ ids, TOut *__restrict__ out, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const TW *row = table + (size_t)ids[t] * table_ld + col0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float z = sum_slices(g, S, slice_stride, (size_t)t * ld + i);
        out[(size_t)t * n + i] = from_f32<TOut>(gelu_tanh_f(z) * to_f32<TW>(row[i]));
    }
}

KESTREL_API int kestrel_gelu_table_mul(const float *g, int S, long long slice_stride, int ld, const void *table, int table_ld, int col0,
                                       const int *ids, void *out, int dtype, int T, int n, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && n > 0 && S > 0, "gelu_table_mul: bad sizes");
    if (dtype == KESTREL_F32)
        kestrel_launch(gelu_table_mul_kernel<float, float>, dim3(T), dim3(128), 0, stream, g, S, (size_t)slice_stride, ld, (const float *)table, table_ld, col0, ids, (float *)out, n);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(gelu_table_mul_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(128), 0, stream, g, S, (size_t)slice_stride, ld, (const __nv_bfloat16 *)table, table_ld, col0, ids,
                       (__nv_bfloat16 *)out, n);
    else
        return kestrel_fail(-2, "gelu_table_mul: unknown dtype %d", dtype);
    return kestrel_check_launch("gelu_table_mul");
}

// ------------------------------------------------------------------------------------------
// y = sum_s p[s, t]; residual[t] += y / sqrt(mean(y^2) + eps) * w.  One block a row, the sum of
// squares in a fixed tree.
// ------------------------------------------------------------------------------------------
#define AN_THREADS 256
__global__ void __launch_bounds__(AN_THREADS)
add_normed_kernel(float *__restrict__ residual, const float *__restrict__ p, int S, size_t slice_stride,
                  const float *__restrict__ w, float eps, int d) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float ys[];
    __shared__ float red[AN_THREADS / 32];
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += AN_THREADS) {
        const float y = sum_slices(p, S, slice_stride, (size_t)t * d + i);
        ys[i] = y;
        ss = fmaf(y, y, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < AN_THREADS / 32; ++k) tot += red[k];
    const float r = 1.0f / sqrtf(tot / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += AN_THREADS) residual[(size_t)t * d + i] += ys[i] * r * w[i];
}

KESTREL_API int kestrel_add_normed(float *residual, const float *p, int S, long long slice_stride, const float *w, float eps, int T, int d,
                                   cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && S > 0 && d <= 12000, "add_normed: bad sizes T=%d d=%d", T, d);
    kestrel_launch(add_normed_kernel, dim3(T), dim3(AN_THREADS), (size_t)d * sizeof(float), stream, residual, p, S, (size_t)slice_stride, w, eps, d);
    return kestrel_check_launch("add_normed");
}

// ------------------------------------------------------------------------------------------
// out[t, i] = sum_s p[s, t, col0 + i] in the storage type, i < n: some columns of a fused
// product, as the input of a second product
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void partial_columns_kernel(const float *__restrict__ p, int S, size_t slice_stride, int ld, int col0,
                                       TOut *__restrict__ out, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t t = idx / n;
    int i = (int)(idx % n);
    out[idx] = from_f32<TOut>(sum_slices(p, S, slice_stride, t * ld + col0 + i));
}

KESTREL_API int kestrel_partial_columns(const float *p, int S, long long slice_stride, int ld, int col0, void *out, int dtype, int T, int n,
                                        cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && n > 0 && S > 0 && col0 >= 0 && col0 + n <= ld, "partial_columns: bad sizes");
    size_t total = (size_t)T * n;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KESTREL_F32)
        kestrel_launch(partial_columns_kernel<float>, dim3(blocks), dim3(256), 0, stream, p, S, (size_t)slice_stride, ld, col0, (float *)out, n, total);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(partial_columns_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, p, S, (size_t)slice_stride, ld, col0, (__nv_bfloat16 *)out, n, total);
    else
        return kestrel_fail(-2, "partial_columns: unknown dtype %d", dtype);
    return kestrel_check_launch("partial_columns");
}
