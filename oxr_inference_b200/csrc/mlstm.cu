// The matrix-memory recurrence of xLSTM (mLSTM) between its in- and out-projections, and the per-head norm with its gate.
//
// Per request and head the state is a matrix S [DK, DV], a vector n [DK] and a running maximum m (all zero for a new
// request; one fp32 row per request: S of every head, then n of every head, then m of every head). With the log input gate
// a_t = cap tanh(zi_t / cap) and the log forget gate b_t = logsigmoid(cap tanh(zf_t / cap)) (zi, zf: the gate projections
// plus their biases):
//
//   m_t = max(b_t + m_(t-1), a_t)
//   S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T          n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                      q_t already scaled by DK^(-1/2)
//
// Gates, exponentials, S, n, m and every sum over them are fp32; T is the activation type of the q|k|v projections.
// The recurrence runs token by token in the order of the sequence whatever the cut, so a position's result does not
// depend on how a prompt was cut into steps. Columns of S (one value dimension each) are independent: a block takes 32
// columns of one head of one request; n and m are the same in all blocks of a head, and the first one writes them back.
#include "common.cuh"

__device__ __forceinline__ float log_sigmoid_f32(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

// grid (ceil(DV / 32), heads, requests); block = 32 * NW threads with NW = ceil(DK / 32). Lane l owns the value column
// p = 32 blockIdx.x + l, warp w the key entries 32 w .. 32 w + 31: a thread keeps 32 entries of S in registers, and entry
// 32 w + l of n. A tile of TT tokens goes through shared memory at a time: k, q, v and the gates are loaded once per tile,
// the warps' partial sums of S^T q and of n . q meet there and are added in the order of the warps after the tile.
template <typename T, int NW, int TT>
__global__ void __launch_bounds__(32 * NW) mlstm_scan_kernel(
    float* __restrict__ y, const T* __restrict__ proj, int proj_stride, int q_col0, int k_col0, int v_col0, const float* __restrict__ gates,
    const float* __restrict__ gate_bias, int heads, int DK, int DV, float cap, float q_scale, float* __restrict__ state, long long slot_stride,
    const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    constexpr int NP = 32 * NW;
    __shared__ __align__(16) float ks[TT][NP];
    __shared__ __align__(16) float qs[TT][NP];
    __shared__ float vs[TT][32], part[TT][NW][32], partn[TT][NW], ga[TT], gb[TT], ms[TT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n = threadIdx.x;
    const int p0 = blockIdx.x * 32, p = p0 + lane, h = blockIdx.y, r = blockIdx.z;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t1 <= t0) return;
    float* slot = state + (long long)state_slots[r] * slot_stride;
    float* S = slot + (long long)h * DK * DV;
    float* nvec = slot + (long long)heads * DK * DV + (long long)h * DK;
    float* mptr = slot + (long long)heads * DK * DV + (long long)heads * DK + h;
    const int n0 = 32 * warp;
    float s[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) s[k] = (n0 + k < DK && p < DV) ? S[(size_t)(n0 + k) * DV + p] : 0.f;
    float nn = n < DK ? nvec[n] : 0.f;
    float m = *mptr;
    const float bias_i = gate_bias[h], bias_f = gate_bias[heads + h];

    for (int tile = t0; tile < t1; tile += TT) {
        const int nt = min(TT, t1 - tile);
        __syncthreads();   // the sums of the tile before have been read
        for (int t = 0; t < nt; ++t) {
            const T* row = proj + (size_t)(tile + t) * proj_stride;
            ks[t][n] = n < DK ? Num<T>::to_f32(row[k_col0 + h * DK + n]) : 0.f;
            qs[t][n] = n < DK ? Num<T>::to_f32(row[q_col0 + h * DK + n]) * q_scale : 0.f;
        }
        for (int i = n; i < nt * 32; i += NP) {
            const int t = i >> 5, c = i & 31;
            vs[t][c] = p0 + c < DV ? Num<T>::to_f32(proj[(size_t)(tile + t) * proj_stride + v_col0 + h * DV + p0 + c]) : 0.f;
        }
        if (n < nt) {
            const float* g = gates + (size_t)(tile + n) * 2 * heads;
            ga[n] = cap * tanhf((g[h] + bias_i) / cap);
            gb[n] = log_sigmoid_f32(cap * tanhf((g[heads + h] + bias_f) / cap));
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float a = ga[t], b = gb[t];
            const float m_new = fmaxf(b + m, a);
            const float keep = expf(b + m - m_new), take = expf(a - m_new);
            m = m_new;
            nn = fmaf(keep, nn, take * ks[t][n]);
            const float nq = warp_sum(nn * qs[t][n]);
            const float tv = take * vs[t][lane];
            const float4* k4 = reinterpret_cast<const float4*>(&ks[t][n0]);
            const float4* q4 = reinterpret_cast<const float4*>(&qs[t][n0]);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};   // four chains, added in a fixed order
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 kk = k4[j], qq = q4[j];
                s[4 * j] = fmaf(keep, s[4 * j], tv * kk.x);
                sum[0] = fmaf(s[4 * j], qq.x, sum[0]);
                s[4 * j + 1] = fmaf(keep, s[4 * j + 1], tv * kk.y);
                sum[1] = fmaf(s[4 * j + 1], qq.y, sum[1]);
                s[4 * j + 2] = fmaf(keep, s[4 * j + 2], tv * kk.z);
                sum[2] = fmaf(s[4 * j + 2], qq.z, sum[2]);
                s[4 * j + 3] = fmaf(keep, s[4 * j + 3], tv * kk.w);
                sum[3] = fmaf(s[4 * j + 3], qq.w, sum[3]);
            }
            part[t][warp][lane] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            if (lane == 0) partn[t][warp] = nq;
            if (n == 0) ms[t] = m;
        }
        __syncthreads();
        for (int i = n; i < nt * 32; i += NP) {
            const int t = i >> 5, c = i & 31;
            if (p0 + c < DV) {
                float num = 0.f, nq = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    num += part[t][w][c];
                    nq += partn[t][w];
                }
                const float den = fmaxf(fabsf(nq), expf(-ms[t])) + 1e-6f;
                y[(size_t)(tile + t) * heads * DV + h * DV + p0 + c] = num / den;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 32; ++k)
        if (n0 + k < DK && p < DV) S[(size_t)(n0 + k) * DV + p] = s[k];
    if (blockIdx.x == 0) {
        if (n < DK) nvec[n] = nn;
        if (n == 0) *mptr = m;
    }
}

OXR_API int oxr_mlstm_scan(float* y, const void* proj, int n_requests, int proj_stride, int q_col0, int k_col0, int v_col0, const float* gates,
                           const float* gate_bias, int heads, int DK, int DV, float cap, float q_scale, float* state, long long slot_stride,
                           const int* cu_q, const int* state_slots, int dtype, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || DK <= 0 || DK > 256 || DV <= 0 || heads > 65535 || n_requests > 65535 || !(cap > 0.f)) return OXR_BAD_ARGUMENT;
    dim3 grid((DV + 31) / 32, heads, n_requests);
    const int nw = (DK + 31) / 32;
#define OXR_MLSTM(T, NW) \
    mlstm_scan_kernel<T, NW, 8><<<grid, 32 * NW, 0, stream>>>(y, (const T*)proj, proj_stride, q_col0, k_col0, v_col0, gates, gate_bias, heads, DK, DV, \
                                                             cap, q_scale, state, slot_stride, cu_q, state_slots)
#define OXR_MLSTM_T(T) \
    do { \
        if (nw <= 1) OXR_MLSTM(T, 1); \
        else if (nw <= 2) OXR_MLSTM(T, 2); \
        else if (nw <= 4) OXR_MLSTM(T, 4); \
        else OXR_MLSTM(T, 8); \
    } while (0)
    if (dtype == 0) OXR_MLSTM_T(float);
    else OXR_MLSTM_T(__nv_bfloat16);
#undef OXR_MLSTM_T
#undef OXR_MLSTM
    return oxr_launch_status();
}

// out[t, h, d] = y[t, h, d] / rms(y[t, h, :]) * weight[h, d] * sigmoid(gate[t, gate_col0 + h DV + d]); one warp per (token, head),
// everything in fp32, rounded once to T.
template <typename T>
__global__ void head_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ gate, int gate_stride, int gate_col0,
                                      const float* __restrict__ weight, int heads, int DV, float eps) {
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * warps + (threadIdx.x >> 5);
    if (h >= heads) return;
    const float* o = y + ((size_t)t * heads + h) * DV;
    float sq = 0.f;
    for (int d = lane; d < DV; d += 32) sq = fmaf(o[d], o[d], sq);
    const float inv = 1.f / sqrtf(warp_sum(sq) / (float)DV + eps);
    for (int d = lane; d < DV; d += 32) {
        const float g = Num<T>::to_f32(gate[(size_t)t * gate_stride + gate_col0 + h * DV + d]);
        out[((size_t)t * heads + h) * DV + d] = Num<T>::from_f32(o[d] * inv * weight[h * DV + d] * (1.f / (1.f + expf(-g))));
    }
}

OXR_API int oxr_head_norm_gate(void* out, const float* y, const void* gate, int n_tokens, int gate_stride, int gate_col0, const float* weight,
                               int heads, int DV, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || DV <= 0) return OXR_BAD_ARGUMENT;
    const int warps = heads >= 4 ? 4 : heads;
    dim3 grid(n_tokens, (heads + warps - 1) / warps);
    if (grid.y > 65535) return OXR_BAD_ARGUMENT;
    if (dtype == 0) head_norm_gate_kernel<float><<<grid, 32 * warps, 0, stream>>>((float*)out, y, (const float*)gate, gate_stride, gate_col0, weight, heads, DV, eps);
    else head_norm_gate_kernel<__nv_bfloat16><<<grid, 32 * warps, 0, stream>>>((__nv_bfloat16*)out, y, (const __nv_bfloat16*)gate, gate_stride, gate_col0, weight, heads, DV, eps);
    return oxr_launch_status();
}
