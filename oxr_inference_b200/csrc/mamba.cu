// A Mamba-2 (state-space duality) mixer's kernels between its in- and out-projection: the short causal convolution
// with SiLU, the roll of the convolution's tail, the selective-state recurrence, and the gated grouped RMSNorm.
//
// A step brings, per request, any number of new tokens (a portion of a prompt, or one decoded token); what earlier steps
// left is the per-request state in a slot: the recurrence's S [heads, vdim, N] and the last taps-1 inputs of the
// convolution [channels, taps-1], both fp32. Everything that enters the recurrence is fp32: dt = softplus(dt + bias)
// (no clamp), the decay exp(-exp(A_log) dt), S itself and the sums over it. T is the activation type of the projections.
//
//   S_t = decay_t S_(t-1) + dt_t B_t x_t^T          y_t = S_t^T C_t + D x_t
//
// The recurrence runs token by token in the order of the sequence whatever the cut, so a position's result does not
// depend on how the prompt was cut into steps. Columns of S (one value dimension p each) are independent: a warp owns
// one column, its lanes the N state entries, and one block takes a few columns of one head of one request.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------- convolution
// out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps-1-j), c]); inputs before the step's first token come from the
// request's tail (oldest first), which is zero for a new request.
template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ proj, int proj_stride, int col0, int channels, int taps,
                                        const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                                        long long slot_stride, const int* __restrict__ req_of_token, const int* __restrict__ cu_q,
                                        const int* __restrict__ state_slots) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= channels) return;
    const int r = req_of_token[t];
    const int i = t - cu_q[r];
    const float* tail = state + (long long)state_slots[r] * slot_stride + (long long)c * (taps - 1);
    float acc = bias[c];
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float v = (i - back >= 0) ? Num<T>::to_f32(proj[(size_t)(t - back) * proj_stride + col0 + c]) : tail[taps - 1 + (i - back)];
        acc = fmaf(w[c * taps + j], v, acc);
    }
    out[(size_t)t * channels + c] = Num<T>::from_f32(acc / (1.f + expf(-acc)));
}

// After the convolution read it: the tail becomes the last taps-1 inputs of (old tail ++ the step's inputs).
template <typename T>
__global__ void conv_tail_roll_kernel(float* __restrict__ state, long long slot_stride, const T* __restrict__ proj, int proj_stride, int col0,
                                      int channels, int taps, const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= channels) return;
    const int t0 = cu_q[r], q = cu_q[r + 1] - t0, keep = taps - 1;
    if (q <= 0) return;
    float* tail = state + (long long)state_slots[r] * slot_stride + (long long)c * keep;
    for (int k = 0; k < keep; ++k) {       // entry k reads entry k + q (not yet overwritten) or a new input
        const int src = q + k - keep;
        tail[k] = src >= 0 ? Num<T>::to_f32(proj[(size_t)(t0 + src) * proj_stride + col0 + c]) : tail[k + q];
    }
}

// ---------------------------------------------------------------------------------------------- recurrence
__device__ __forceinline__ float softplus_f32(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// grid (ceil(vdim / WARPS), heads, requests); warp w owns column p = blockIdx.x * WARPS + w; lane l holds S[p, l + 32 k].
template <typename T, int NPL, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) ssm_scan_kernel(
    float* __restrict__ y, const T* __restrict__ xbc, const T* __restrict__ proj, int proj_stride, int dt_col0, int heads, int vdim, int N,
    int groups, const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state,
    long long slot_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.x * WARPS + warp, h = blockIdx.y, r = blockIdx.z;
    if (p >= vdim) return;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t1 <= t0) return;
    const int inner = heads * vdim, channels = inner + 2 * groups * N, g = h / (heads / groups);
    float* S = state + (long long)state_slots[r] * slot_stride + ((long long)h * vdim + p) * N;
    float s[NPL];
#pragma unroll
    for (int k = 0; k < NPL; ++k) s[k] = (lane + 32 * k < N) ? S[lane + 32 * k] : 0.f;
    const float neg_a = -expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
    const int x_col = h * vdim + p, b_col = inner + g * N, c_col = inner + groups * N + g * N;

    // the next token's inputs are fetched while this token's sums run
    float dt_raw = Num<T>::to_f32(proj[(size_t)t0 * proj_stride + dt_col0 + h]);
    float x = Num<T>::to_f32(xbc[(size_t)t0 * channels + x_col]);
    float b[NPL], c[NPL];
#pragma unroll
    for (int k = 0; k < NPL; ++k) {
        const int n = lane + 32 * k;
        b[k] = n < N ? Num<T>::to_f32(xbc[(size_t)t0 * channels + b_col + n]) : 0.f;
        c[k] = n < N ? Num<T>::to_f32(xbc[(size_t)t0 * channels + c_col + n]) : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
        const float dt_now = dt_raw, x_now = x;
        float b_now[NPL], c_now[NPL];
#pragma unroll
        for (int k = 0; k < NPL; ++k) { b_now[k] = b[k]; c_now[k] = c[k]; }
        if (t + 1 < t1) {
            dt_raw = Num<T>::to_f32(proj[(size_t)(t + 1) * proj_stride + dt_col0 + h]);
            x = Num<T>::to_f32(xbc[(size_t)(t + 1) * channels + x_col]);
#pragma unroll
            for (int k = 0; k < NPL; ++k) {
                const int n = lane + 32 * k;
                if (n < N) {
                    b[k] = Num<T>::to_f32(xbc[(size_t)(t + 1) * channels + b_col + n]);
                    c[k] = Num<T>::to_f32(xbc[(size_t)(t + 1) * channels + c_col + n]);
                }
            }
        }
        const float dt = softplus_f32(dt_now + bias);
        const float decay = expf(neg_a * dt);
        const float dx = dt * x_now;
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            s[k] = fmaf(decay, s[k], dx * b_now[k]);
            part = fmaf(s[k], c_now[k], part);
        }
        part = warp_sum(part);
        if (lane == 0) y[(size_t)t * inner + x_col] = fmaf(skip, x_now, part);
    }
#pragma unroll
    for (int k = 0; k < NPL; ++k)
        if (lane + 32 * k < N) S[lane + 32 * k] = s[k];
}

// ---------------------------------------------------------------------------------------------- gated grouped norm
// v = y * silu(z); out = v * rsqrt(mean over the part of v^2 + eps) * weight. grid (parts, tokens).
template <typename T>
__global__ void gated_group_norm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ proj, int proj_stride, int z_col0,
                                        const float* __restrict__ weight, int inner, int part, float eps) {
    __shared__ float red[32];
    const int t = blockIdx.y, lo = blockIdx.x * part;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float z = Num<T>::to_f32(proj[(size_t)t * proj_stride + z_col0 + lo + i]);
        const float v = y[(size_t)t * inner + lo + i] * (z / (1.f + expf(-z)));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float z = Num<T>::to_f32(proj[(size_t)t * proj_stride + z_col0 + lo + i]);
        const float v = y[(size_t)t * inner + lo + i] * (z / (1.f + expf(-z)));
        out[(size_t)t * inner + lo + i] = Num<T>::from_f32(v * inv * weight[lo + i]);
    }
}

// ---------------------------------------------------------------------------------------------- launchers
// proj: the in-projection's output [tokens, proj_stride], columns [z: inner | x, B, C: channels | dt: heads].
template <typename T>
static int mamba_conv(void* out, const void* proj, int n_tokens, int n_requests, int proj_stride, int col0, int channels, int taps,
                      const float* w, const float* bias, float* state, long long slot_stride, const int* req_of_token, const int* cu_q,
                      const int* state_slots, cudaStream_t stream) {
    dim3 grid((channels + 127) / 128, n_tokens);
    causal_conv_silu_kernel<T><<<grid, 128, 0, stream>>>((T*)out, (const T*)proj, proj_stride, col0, channels, taps, w, bias, state, slot_stride,
                                                        req_of_token, cu_q, state_slots);
    if (taps > 1) {
        dim3 grid2((channels + 127) / 128, n_requests);
        conv_tail_roll_kernel<T><<<grid2, 128, 0, stream>>>(state, slot_stride, (const T*)proj, proj_stride, col0, channels, taps, cu_q, state_slots);
    }
    return oxr_launch_status();
}

OXR_API int oxr_mamba_conv(void* out, const void* proj, int n_tokens, int n_requests, int proj_stride, int col0, int channels, int taps,
                           const float* w, const float* bias, float* state, long long slot_stride, const int* req_of_token, const int* cu_q,
                           const int* state_slots, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (channels <= 0 || taps < 1 || n_tokens > 65535 * 64 || n_requests > 65535) return OXR_BAD_ARGUMENT;
    if (n_tokens > 65535) return OXR_BAD_ARGUMENT;
    return dtype == 0 ? mamba_conv<float>(out, proj, n_tokens, n_requests, proj_stride, col0, channels, taps, w, bias, state, slot_stride, req_of_token,
                                          cu_q, state_slots, stream)
                      : mamba_conv<__nv_bfloat16>(out, proj, n_tokens, n_requests, proj_stride, col0, channels, taps, w, bias, state, slot_stride,
                                                  req_of_token, cu_q, state_slots, stream);
}

template <typename T, int NPL>
static void mamba_scan(float* y, const void* xbc, const void* proj, int n_requests, int proj_stride, int dt_col0, int heads, int vdim, int N, int groups,
                       const float* dt_bias, const float* a_log, const float* d_skip, float* state, long long slot_stride, const int* cu_q,
                       const int* state_slots, cudaStream_t stream) {
    constexpr int WARPS = 4;
    dim3 grid((vdim + WARPS - 1) / WARPS, heads, n_requests);
    ssm_scan_kernel<T, NPL, WARPS><<<grid, 32 * WARPS, 0, stream>>>(y, (const T*)xbc, (const T*)proj, proj_stride, dt_col0, heads, vdim, N, groups, dt_bias,
                                                                    a_log, d_skip, state, slot_stride, cu_q, state_slots);
}

OXR_API int oxr_mamba_scan(float* y, const void* xbc, const void* proj, int n_requests, int proj_stride, int dt_col0, int heads, int vdim, int N, int groups,
                           const float* dt_bias, const float* a_log, const float* d_skip, float* state, long long slot_stride, const int* cu_q,
                           const int* state_slots, int dtype, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || N <= 0 || N > 256 || groups <= 0 || heads % groups || n_requests > 65535 || heads > 65535) return OXR_BAD_ARGUMENT;
    const int npl = (N + 31) / 32;
#define OXR_SCAN(NPL) \
    (dtype == 0 ? mamba_scan<float, NPL>(y, xbc, proj, n_requests, proj_stride, dt_col0, heads, vdim, N, groups, dt_bias, a_log, d_skip, state, \
                                         slot_stride, cu_q, state_slots, stream) \
                : mamba_scan<__nv_bfloat16, NPL>(y, xbc, proj, n_requests, proj_stride, dt_col0, heads, vdim, N, groups, dt_bias, a_log, d_skip, state, \
                                                 slot_stride, cu_q, state_slots, stream))
    if (npl <= 1) OXR_SCAN(1);
    else if (npl <= 2) OXR_SCAN(2);
    else if (npl <= 4) OXR_SCAN(4);
    else OXR_SCAN(8);
#undef OXR_SCAN
    return oxr_launch_status();
}

OXR_API int oxr_gated_group_norm(void* out, const float* y, const void* proj, int n_tokens, int proj_stride, int z_col0, const float* weight, int inner,
                                 int parts, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (inner <= 0 || parts <= 0 || inner % parts || n_tokens > 65535) return OXR_BAD_ARGUMENT;
    const int part = inner / parts;
    const int threads = part >= 1024 ? 256 : 128;
    dim3 grid(parts, n_tokens);
    if (dtype == 0) gated_group_norm_kernel<float><<<grid, threads, 0, stream>>>((float*)out, y, (const float*)proj, proj_stride, z_col0, weight, inner, part, eps);
    else gated_group_norm_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)out, y, (const __nv_bfloat16*)proj, proj_stride, z_col0, weight,
                                                                              inner, part, eps);
    return oxr_launch_status();
}
