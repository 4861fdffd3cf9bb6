// A Mamba-2 (state-space duality) mixer's kernels between its in- and out-projection: the short causal convolution
// with SiLU, the roll of the convolution's tail, the selective-state recurrence, and the gated grouped RMSNorm.
//
// A step brings, per request, any number of new tokens (a portion of a prompt, or one decoded token); what earlier steps
// left is the per-request state in a slot: the recurrence's S [heads, N, vdim] and the last taps-1 inputs of the
// convolution [channels, taps-1], both fp32. Everything that enters the recurrence is fp32: dt = softplus(dt + bias)
// (no clamp), the decay exp(-exp(A_log) dt), S itself and the sums over it. T is the activation type of the projections.
//
//   S_t = decay_t S_(t-1) + dt_t B_t x_t^T          y_t = S_t^T C_t + D x_t
//
// The recurrence runs token by token in the order of the sequence whatever the cut, so a position's result does not
// depend on how the prompt was cut into steps. Columns of S (one value dimension p each) are independent: a block takes
// 32 columns of one head of one request.
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

// grid (ceil(vdim / 32), heads, requests); block = 32 * NW threads with NW = ceil(N / 32). Lane l owns the value column
// p = 32 blockIdx.x + l, warp w the state entries n = 32 w .. 32 w + 31, so a thread keeps 32 entries of S in registers and
// updates them with plain multiply-adds: B and C of a token are the same for all lanes and come from shared memory as
// broadcast 16-byte loads, no shuffles. The step's tokens go through shared memory TT at a time (B, C, x, softplus and decay,
// each computed once per token and block; the next tile is fetched while this one is computed); the warps' partial sums of y
// meet there too and are added in the order of the warps.
// S is stored [heads, N, vdim]: the lanes of a warp read and write 128 contiguous bytes per state entry.
template <typename T, int NW, int TT>
__global__ void __launch_bounds__(32 * NW) ssm_scan_kernel(
    float* __restrict__ y, const T* __restrict__ xbc, const T* __restrict__ proj, int proj_stride, int dt_col0, int heads, int vdim, int N,
    int groups, const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state,
    long long slot_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    constexpr int NP = 32 * NW;                       // N rounded up to whole warps
    extern __shared__ __align__(16) float scan_smem[];
    float* Bs = scan_smem;                            // [TT][NP]
    float* Cs = Bs + TT * NP;                         // [TT][NP]
    float* xs = Cs + TT * NP;                         // [TT][32]
    float* part = xs + TT * 32;                       // [TT][NW][32]
    float* dts = part + TT * NW * 32;                 // [TT]
    float* decays = dts + TT;                         // [TT]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p0 = blockIdx.x * 32, p = p0 + lane, h = blockIdx.y, r = blockIdx.z;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t1 <= t0) return;
    const int inner = heads * vdim, channels = inner + 2 * groups * N, g = h / (heads / groups);
    const int b_col = inner + g * N, c_col = inner + groups * N + g * N, n0 = 32 * warp;
    float* S = state + (long long)state_slots[r] * slot_stride + (long long)h * N * vdim;
    float s[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) s[k] = (n0 + k < N && p < vdim) ? S[(size_t)(n0 + k) * vdim + p] : 0.f;
    const float neg_a = -expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];

    // A tile's inputs are fetched into registers while the tile before it is computed (all loads of a tile are issued back to
    // back: one trip to memory per tile, hidden behind the sums), then written to shared memory between two barriers.
    constexpr int XPT = (TT + NW - 1) / NW;           // x values per thread and tile
    const int n = threadIdx.x;                        // this thread's state entry in the fetch (NP threads, NP entries)
    T bv[TT], cv[TT], xv[XPT], dtv = Num<T>::from_f32(0.f);
    auto fetch = [&](int tile) {
        const int nt = min(TT, t1 - tile);
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const bool ok = t < nt && n < N;
            const T* row = xbc + (size_t)(tile + (t < nt ? t : 0)) * channels;
            bv[t] = ok ? row[b_col + n] : Num<T>::from_f32(0.f);
            cv[t] = ok ? row[c_col + n] : Num<T>::from_f32(0.f);
        }
#pragma unroll
        for (int j = 0; j < XPT; ++j) {
            const int i = threadIdx.x + j * 32 * NW, t = i >> 5, c = i & 31;
            xv[j] = (t < nt && p0 + c < vdim) ? xbc[(size_t)(tile + t) * channels + h * vdim + p0 + c] : Num<T>::from_f32(0.f);
        }
        if ((int)threadIdx.x < nt) dtv = proj[(size_t)(tile + threadIdx.x) * proj_stride + dt_col0 + h];
    };
    auto stash = [&](int tile) {
        const int nt = min(TT, t1 - tile);
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            Bs[t * NP + n] = Num<T>::to_f32(bv[t]);
            Cs[t * NP + n] = Num<T>::to_f32(cv[t]);
        }
#pragma unroll
        for (int j = 0; j < XPT; ++j) {
            const int i = threadIdx.x + j * 32 * NW;
            if (i < TT * 32) xs[i] = Num<T>::to_f32(xv[j]);
        }
        if ((int)threadIdx.x < nt) {
            const float dt = softplus_f32(Num<T>::to_f32(dtv) + bias);
            dts[threadIdx.x] = dt;
            decays[threadIdx.x] = expf(neg_a * dt);
        }
    };
    fetch(t0);
    stash(t0);
    __syncthreads();
    for (int tile = t0; tile < t1; tile += TT) {
        const int nt = min(TT, t1 - tile);
        const bool more = tile + TT < t1;
        if (more) fetch(tile + TT);
        for (int t = 0; t < nt; ++t) {
            const float decay = decays[t], dx = dts[t] * xs[t * 32 + lane];
            const float4* b4 = reinterpret_cast<const float4*>(Bs + t * NP + n0);
            const float4* c4 = reinterpret_cast<const float4*>(Cs + t * NP + n0);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};   // four chains instead of one of 32 dependent multiply-adds; added in a fixed order
#pragma unroll
            for (int k4 = 0; k4 < 8; ++k4) {
                const float4 b = b4[k4], c = c4[k4];
                s[4 * k4] = fmaf(decay, s[4 * k4], dx * b.x);
                sum[0] = fmaf(s[4 * k4], c.x, sum[0]);
                s[4 * k4 + 1] = fmaf(decay, s[4 * k4 + 1], dx * b.y);
                sum[1] = fmaf(s[4 * k4 + 1], c.y, sum[1]);
                s[4 * k4 + 2] = fmaf(decay, s[4 * k4 + 2], dx * b.z);
                sum[2] = fmaf(s[4 * k4 + 2], c.z, sum[2]);
                s[4 * k4 + 3] = fmaf(decay, s[4 * k4 + 3], dx * b.w);
                sum[3] = fmaf(s[4 * k4 + 3], c.w, sum[3]);
            }
            part[(t * NW + warp) * 32 + lane] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 32; i += 32 * NW) {
            const int t = i >> 5, c = i & 31;
            if (p0 + c >= vdim) continue;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) v += part[(t * NW + w) * 32 + c];
            y[(size_t)(tile + t) * inner + h * vdim + p0 + c] = fmaf(skip, xs[i], v);
        }
        if (!more) break;
        __syncthreads();   // everyone has read this tile's buffers
        stash(tile + TT);
        __syncthreads();
    }
    if (p < vdim) {
#pragma unroll
        for (int k = 0; k < 32; ++k)
            if (n0 + k < N) S[(size_t)(n0 + k) * vdim + p] = s[k];
    }
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

template <typename T, int NW>
static void mamba_scan(float* y, const void* xbc, const void* proj, int n_requests, int proj_stride, int dt_col0, int heads, int vdim, int N, int groups,
                       const float* dt_bias, const float* a_log, const float* d_skip, float* state, long long slot_stride, const int* cu_q,
                       const int* state_slots, cudaStream_t stream) {
    constexpr int TT = NW <= 4 ? 16 : 8;
    constexpr size_t smem = (size_t)(TT * (2 * 32 * NW + 32 + NW * 32 + 2)) * sizeof(float);
    static_assert(smem <= 48 * 1024, "the tile fits the default shared memory");
    dim3 grid((vdim + 31) / 32, heads, n_requests);
    ssm_scan_kernel<T, NW, TT><<<grid, 32 * NW, smem, stream>>>(y, (const T*)xbc, (const T*)proj, proj_stride, dt_col0, heads, vdim, N, groups, dt_bias,
                                                                a_log, d_skip, state, slot_stride, cu_q, state_slots);
}

OXR_API int oxr_mamba_scan(float* y, const void* xbc, const void* proj, int n_requests, int proj_stride, int dt_col0, int heads, int vdim, int N, int groups,
                           const float* dt_bias, const float* a_log, const float* d_skip, float* state, long long slot_stride, const int* cu_q,
                           const int* state_slots, int dtype, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || N <= 0 || N > 256 || groups <= 0 || heads % groups || n_requests > 65535 || heads > 65535) return OXR_BAD_ARGUMENT;
    const int nw = (N + 31) / 32;
#define OXR_SCAN(NW) \
    (dtype == 0 ? mamba_scan<float, NW>(y, xbc, proj, n_requests, proj_stride, dt_col0, heads, vdim, N, groups, dt_bias, a_log, d_skip, state, \
                                        slot_stride, cu_q, state_slots, stream) \
                : mamba_scan<__nv_bfloat16, NW>(y, xbc, proj, n_requests, proj_stride, dt_col0, heads, vdim, N, groups, dt_bias, a_log, d_skip, state, \
                                                slot_stride, cu_q, state_slots, stream))
    switch (nw) {
        case 1: OXR_SCAN(1); break;
        case 2: OXR_SCAN(2); break;
        case 3: OXR_SCAN(3); break;
        case 4: OXR_SCAN(4); break;
        case 5: OXR_SCAN(5); break;
        case 6: OXR_SCAN(6); break;
        case 7: OXR_SCAN(7); break;
        default: OXR_SCAN(8); break;
    }
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
