// A recurrent mixer: the gated delta rule with one decay per key channel, and the short causal
// convolutions in front of it.  Per head, with a state S [d, dv] that starts at zero and is
// carried from token to token of a request (float32, in the request's state slot):
//
//     S <- diag(a_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// The read-out sees the token's own write.  Everything that enters the recurrence is float32.
//
// Kernels, in the order of a step:
//   conv_silu     y[t, c] = silu(sum_j w[c, j] x[t - (taps-1) + j, c]) per channel of the fused
//                 q|k|v product; inputs before this step's first token of a request come from the
//                 request's state slot (the last taps-1 inputs; zeros for a new request)
//   conv_tail     writes the last taps-1 inputs back to the slot
//   gates         q, k made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q scaled by d^-1/2;
//                 beta = sigmoid(.); a = exp(-exp(A_log[h]) softplus(. + dt_bias))
//   scan          the recurrence; a warp takes 32 value columns of one (request, head): column j
//                 of S stays in the registers of lane j, so S^T k and S^T q are sums inside a
//                 thread, in ascending key channel - a token's result does not depend on how the
//                 request was cut into steps or on the batch
//   out_norm_gate o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) per head, in the storage type
#include "common.cuh"
#include <math.h>

#define DR_MAX_TAPS 8

// sum of a product's slices at (token, column)
__device__ __forceinline__ float slices_at(const float *p, int S, size_t slice_stride, size_t off) {
    float v = 0.f;
    for (int s = 0; s < S; ++s) v += p[(size_t)s * slice_stride + off];
    return v;
}

__global__ void delta_conv_silu_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, const float *__restrict__ w,
                                       int taps, const float *__restrict__ state, size_t state_stride, size_t tail_off,
                                       const int *__restrict__ seq_of_token, const int *__restrict__ cu_seqlens,
                                       const int *__restrict__ slots, float *__restrict__ out, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = cu_seqlens[seq];
    const int i = t - first;
    const float *tail = state + (size_t)slots[seq] * state_stride + tail_off;     // [taps - 1][C], oldest first
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float y = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int n = i - (taps - 1) + j;          // input index among this step's tokens of the request
            const float x = n >= 0 ? slices_at(partial, S, slice_stride, (size_t)(first + n) * ld + c)
                                   : tail[(size_t)(taps - 1 + n) * C + c];
            y = fmaf(w[(size_t)c * taps + j], x, y);
        }
        out[(size_t)t * C + c] = y / (1.0f + expf(-y));
    }
}

__global__ void delta_conv_tail_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, int taps,
                                       float *__restrict__ state, size_t state_stride, size_t tail_off,
                                       const int *__restrict__ cu_seqlens, const int *__restrict__ slots, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x;
    const int first = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - first;
    float *tail = state + (size_t)slots[seq] * state_stride + tail_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float keep[DR_MAX_TAPS];
#pragma unroll
        for (int r = 0; r < DR_MAX_TAPS; ++r) {
            if (r < taps - 1) {
                const int n = n_tok - (taps - 1) + r;
                keep[r] = n >= 0 ? slices_at(partial, S, slice_stride, (size_t)(first + n) * ld + c)
                                 : tail[(size_t)(taps - 1 + n) * C + c];
            }
        }
#pragma unroll
        for (int r = 0; r < DR_MAX_TAPS; ++r)
            if (r < taps - 1) tail[(size_t)r * C + c] = keep[r];
    }
}

// act [T, C] = q (G*d) | k (G*d) | v (H*dv) after convolution and silu
__global__ void __launch_bounds__(128)
delta_gates_kernel(const float *__restrict__ act, int C, const float *__restrict__ partial, int S, size_t slice_stride, int ld, int col_beta,
                   const float *__restrict__ a_part, int Sa, size_t a_stride, const float *__restrict__ A_log,
                   const float *__restrict__ dt_bias, float *__restrict__ qn, float *__restrict__ kn, float *__restrict__ decay,
                   float *__restrict__ beta, int H, int G, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float q_scale = 1.0f / sqrtf((float)d);
    for (int r = warp; r < 2 * G; r += 4) {                // q heads, then k heads
        const float *x = act + (size_t)t * C + (size_t)r * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float mul = (1.0f / sqrtf(ss + 1e-6f)) * (r < G ? q_scale : 1.0f);
        float *dst = r < G ? qn + ((size_t)t * G + r) * d : kn + ((size_t)t * G + (r - G)) * d;
        for (int i = lane; i < d; i += 32) dst[i] = x[i] * mul;
    }
    for (int idx = threadIdx.x; idx < H * d; idx += 128) {
        const int h = idx / d;
        const float a = slices_at(a_part, Sa, a_stride, (size_t)t * H * d + idx) + dt_bias[idx];
        const float sp = a > 20.f ? a : log1pf(expf(a));
        decay[(size_t)t * H * d + idx] = expf(-expf(A_log[h]) * sp);
    }
    for (int h = threadIdx.x; h < H; h += 128) {
        const float z = slices_at(partial, S, slice_stride, (size_t)t * ld + col_beta + h);
        beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-z));
    }
}

#define DR_TC 4        // tokens staged in shared memory at a time

template <int D>
__global__ void __launch_bounds__(32)
delta_scan_kernel(const float *__restrict__ qn, const float *__restrict__ kn, const float *__restrict__ decay,
                  const float *__restrict__ act, int C, int col_v, const float *__restrict__ beta, float *__restrict__ state,
                  size_t state_stride, const int *__restrict__ cu_seqlens, const int *__restrict__ slots,
                  float *__restrict__ out, int H, int G, int d, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sk[DR_TC][D], sq[DR_TC][D], sa[DR_TC][D];
    const int lane = threadIdx.x;
    const int j = blockIdx.x * 32 + lane, h = blockIdx.y, seq = blockIdx.z;
    const int g = h / (H / G);
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    const bool live = j < dv;
    float *Sg = state + (size_t)slots[seq] * state_stride + (size_t)h * d * dv;     // [d][dv]
    float Sc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) Sc[i] = (i < d && live) ? Sg[(size_t)i * dv + j] : 0.f;
    for (int tb = t0; tb < t1; tb += DR_TC) {
        const int n = min(DR_TC, t1 - tb);
        __syncwarp();
        for (int idx = lane; idx < DR_TC * D; idx += 32) {
            const int c = idx / D, i = idx % D;
            const bool ok = c < n && i < d;
            sk[c][i] = ok ? kn[((size_t)(tb + c) * G + g) * d + i] : 0.f;
            sq[c][i] = ok ? qn[((size_t)(tb + c) * G + g) * d + i] : 0.f;
            sa[c][i] = ok ? decay[((size_t)(tb + c) * H + h) * d + i] : 1.f;
        }
        __syncwarp();
        for (int c = 0; c < n; ++c) {
            const int t = tb + c;
            const float v = live ? act[(size_t)t * C + col_v + (size_t)h * dv + j] : 0.f;
            const float b = beta[(size_t)t * H + h];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) {
                Sc[i] *= sa[c][i];
                acc = fmaf(Sc[i], sk[c][i], acc);
            }
            const float u = b * (v - acc);
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) {
                Sc[i] = fmaf(sk[c][i], u, Sc[i]);
                o = fmaf(Sc[i], sq[c][i], o);
            }
            if (live) out[((size_t)t * H + h) * dv + j] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < D; ++i)
            if (i < d) Sg[(size_t)i * dv + j] = Sc[i];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
delta_out_kernel(const float *__restrict__ o, const float *__restrict__ w, float eps, const float *__restrict__ g_part, int Sg,
                 size_t g_stride, T *__restrict__ out, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < H; h += 4) {
        const size_t base = ((size_t)t * H + h) * dv;
        float ss = 0.f;
        for (int i = lane; i < dv; i += 32) ss = fmaf(o[base + i], o[base + i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int i = lane; i < dv; i += 32) {
            const float z = slices_at(g_part, Sg, g_stride, base + i);
            out[base + i] = from_f32<T>(o[base + i] * r * w[i] * (1.0f / (1.0f + expf(-z))));
        }
    }
}

KESTREL_API int kestrel_delta_conv_silu(const float *partial, int S, long long slice_stride, int ld, const float *w, int taps, float *state,
                                        long long state_stride, long long tail_off, const int *seq_of_token, const int *cu_seqlens,
                                        const int *slots, float *out, int T, int nseq, int C, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && nseq > 0 && C > 0 && S > 0 && taps >= 1 && taps <= DR_MAX_TAPS + 1, "delta_conv_silu: bad sizes (taps %d)", taps);
    kestrel_launch(delta_conv_silu_kernel, dim3(T), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, w, taps, (const float *)state,
                   (size_t)state_stride, (size_t)tail_off, seq_of_token, cu_seqlens, slots, out, C);
    int rc = kestrel_check_launch("delta_conv_silu");
    if (rc != 0 || taps == 1) return rc;
    kestrel_launch(delta_conv_tail_kernel, dim3(nseq, (C + 255) / 256), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, taps, state,
                   (size_t)state_stride, (size_t)tail_off, cu_seqlens, slots, C);
    return kestrel_check_launch("delta_conv_tail");
}

KESTREL_API int kestrel_delta_gates(const float *act, int C, const float *partial, int S, long long slice_stride, int ld, int col_beta,
                                    const float *a_part, int Sa, long long a_stride, const float *A_log, const float *dt_bias, float *qn,
                                    float *kn, float *decay, float *beta, int T, int H, int G, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && d > 0, "delta_gates: bad sizes");
    kestrel_launch(delta_gates_kernel, dim3(T), dim3(128), 0, stream, act, C, partial, S, (size_t)slice_stride, ld, col_beta, a_part, Sa,
                   (size_t)a_stride, A_log, dt_bias, qn, kn, decay, beta, H, G, d);
    return kestrel_check_launch("delta_gates");
}

KESTREL_API int kestrel_delta_scan(const float *qn, const float *kn, const float *decay, const float *act, int C, int col_v, const float *beta,
                                   float *state, long long state_stride, const int *cu_seqlens, const int *slots, float *out, int nseq,
                                   int H, int G, int d, int dv, cudaStream_t stream) {
    if (nseq == 0) return 0;
    KESTREL_REQUIRE(nseq > 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "delta_scan: bad sizes");
    KESTREL_REQUIRE(d <= 256, "delta_scan: key size %d exceeds 256", d);
    KESTREL_REQUIRE(H <= 65535 && nseq <= 65535, "delta_scan: grid too large");
    dim3 grid((dv + 31) / 32, H, nseq);
#define DR_LAUNCH(D)                                                                                                                  \
    kestrel_launch(delta_scan_kernel<D>, grid, dim3(32), 0, stream, qn, kn, decay, act, C, col_v, beta, state, (size_t)state_stride, \
                   cu_seqlens, slots, out, H, G, d, dv)
    if (d <= 32) DR_LAUNCH(32);
    else if (d <= 64) DR_LAUNCH(64);
    else if (d <= 128) DR_LAUNCH(128);
    else DR_LAUNCH(256);
#undef DR_LAUNCH
    return kestrel_check_launch("delta_scan");
}

KESTREL_API int kestrel_delta_out(const float *o, const float *w, float eps, const float *g_part, int Sg, long long g_stride, void *out,
                                  int dtype, int T, int H, int dv, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && dv > 0 && Sg > 0, "delta_out: bad sizes");
    if (dtype == KESTREL_F32)
        kestrel_launch(delta_out_kernel<float>, dim3(T), dim3(128), 0, stream, o, w, eps, g_part, Sg, (size_t)g_stride, (float *)out, H, dv);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(delta_out_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, o, w, eps, g_part, Sg, (size_t)g_stride, (__nv_bfloat16 *)out, H, dv);
    else
        return kestrel_fail(-2, "delta_out: unknown dtype %d", dtype);
    return kestrel_check_launch("delta_out");
}
