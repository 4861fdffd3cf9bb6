// What stands between the q|k|v projection and the attention kernel in a mixer whose projections have biases and pass a
// short causal convolution over time: ONE kernel adds the biases, filters every channel, scales the queries by a
// temperature that grows with the position, blends the values with those another layer kept for the same tokens, and
// writes keys and values to their cache slots. A second, small kernel rolls each request's convolution tail forward.
//
//   u_t = proj_t + bias                      (zero before a sequence's start)
//   y_t[c] = sum_j w[c, j] u_(t - taps + 1 + j)[c]
//   q_t = y_t[q columns] * (1 + coef ln(floor((p + 1) / every) + 1))          p: the token's position
//   v_t = (1 - lambda) y_t[v columns] + lambda first_t                        when the layer blends
//
// A step brings, per request, any number of new tokens; the last taps-1 values of u of each request live in its state
// slot (fp32, [channels, taps-1], oldest first; zero for a new request, which is what "zero before the start" needs).
// Sums, the temperature and the blend are fp32; T is the type of the projection, the queries and the cache.
//
// Also here: a bias row added to a matrix in place and an fp32 matrix scaled in place.
#include "common.cuh"

// Per-head widths: q and k heads have dk entries, v heads dv; in memory a q head takes qw entries, a cached key head kw and a cached
// value head vw (wider than dk / dv when the cache pads keys and values to one size for the tiled attention kernels; the padding
// is never written and stays zero).
struct HeadWidths {
    int dk, dv, qw, kw, vw;
};

template <typename T>
__global__ void conv_qkv_store_kernel(
    T* __restrict__ q_out, T* __restrict__ v_out, const T* __restrict__ proj, int proj_stride, int cq, int ck, int cv, int taps,
    const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ tails, long long slot_stride,
    const int* __restrict__ req_of_token, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
    const int* __restrict__ positions, float temp_coef, int temp_every, const float* __restrict__ blend, const T* __restrict__ first,
    T* __restrict__ k_pool, T* __restrict__ v_pool, const int* __restrict__ slots, long long n_slots, int* status, const HeadWidths hw) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    const int channels = cq + ck + cv;
    if (c >= channels) return;
    const int r = req_of_token[t];
    const int i = t - cu_q[r];
    const float b = bias != nullptr ? bias[c] : 0.f;
    float acc;
    if (taps <= 0) {
        acc = Num<T>::to_f32(proj[(size_t)t * proj_stride + c]) + b;
    } else {
        const float* tail = tails + (long long)state_slots[r] * slot_stride + (long long)c * (taps - 1);
        acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;
            const float u = (i - back >= 0) ? Num<T>::to_f32(proj[(size_t)(t - back) * proj_stride + c]) + b : tail[taps - 1 + (i - back)];
            acc = fmaf(w[c * taps + j], u, acc);
        }
    }
    if (c < cq) {
        if (temp_every > 0) acc *= 1.f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
        q_out[(size_t)t * (cq / hw.dk) * hw.qw + (c / hw.dk) * hw.qw + c % hw.dk] = Num<T>::from_f32(acc);
        return;
    }
    const long long slot = slots[t];
    if (slot >= n_slots) oxr_report(status, OXR_BAD_SLOT, t);
    const bool store = slot >= 0 && slot < n_slots;
    if (c < cq + ck) {
        const int kc = c - cq;
        if (store) k_pool[slot * (ck / hw.dk) * hw.kw + (kc / hw.dk) * hw.kw + kc % hw.dk] = Num<T>::from_f32(acc);
        return;
    }
    const int cc = c - cq - ck;
    if (blend != nullptr) {
        const float lam = blend[0];
        acc = (1.f - lam) * acc + lam * Num<T>::to_f32(first[(size_t)t * cv + cc]);
    }
    const T rounded = Num<T>::from_f32(acc);
    if (v_out != nullptr) v_out[(size_t)t * cv + cc] = rounded;
    if (store) v_pool[slot * (cv / hw.dv) * hw.vw + (cc / hw.dv) * hw.vw + cc % hw.dv] = rounded;
}


struct __align__(16) Bf16x8 { __nv_bfloat162 v[4]; };

// What happens to 8 neighbouring filtered channels of token t: queries get their temperature and go to q_out; keys go to their
// cache slot; values are blended, kept for later layers if asked, and go to their cache slot.
__device__ __forceinline__ void conv_finish8(float* acc, int c, int t, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ v_out, int cq,
                                             int ck, int cv, const int* __restrict__ positions, float temp_coef, int temp_every,
                                             const float* __restrict__ blend, const __nv_bfloat16* __restrict__ first,
                                             __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ slots,
                                             long long n_slots, int* status, const HeadWidths& hw) {
    auto pack = [&](const float* x) {
        Bf16x8 out;
#pragma unroll
        for (int k = 0; k < 4; ++k) out.v[k] = __floats2bfloat162_rn(x[2 * k], x[2 * k + 1]);
        return out;
    };
    if (c < cq) {
        if (temp_every > 0) {
            const float f = 1.f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] *= f;
        }
        *reinterpret_cast<Bf16x8*>(q_out + (size_t)t * (cq / hw.dk) * hw.qw + (c / hw.dk) * hw.qw + c % hw.dk) = pack(acc);
        return;
    }
    const long long slot = slots[t];
    if (slot >= n_slots) oxr_report(status, OXR_BAD_SLOT, t);
    const bool store = slot >= 0 && slot < n_slots;
    if (c < cq + ck) {
        const int kc = c - cq;
        if (store) *reinterpret_cast<Bf16x8*>(k_pool + slot * (ck / hw.dk) * hw.kw + (kc / hw.dk) * hw.kw + kc % hw.dk) = pack(acc);
        return;
    }
    const int cc = c - cq - ck;
    if (blend != nullptr) {
        const float lam = blend[0];
        const Bf16x8 raw = *reinterpret_cast<const Bf16x8*>(first + (size_t)t * cv + cc);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(raw.v[k]);
            acc[2 * k] = (1.f - lam) * acc[2 * k] + lam * f.x;
            acc[2 * k + 1] = (1.f - lam) * acc[2 * k + 1] + lam * f.y;
        }
    }
    const Bf16x8 rounded = pack(acc);
    if (v_out != nullptr) *reinterpret_cast<Bf16x8*>(v_out + (size_t)t * cv + cc) = rounded;
    if (store) *reinterpret_cast<Bf16x8*>(v_pool + slot * (cv / hw.dv) * hw.vw + (cc / hw.dv) * hw.vw + cc % hw.dv) = rounded;
}

// The same for bfloat16 with 16-byte accesses: a thread takes 8 neighbouring channels (all of q, of k or of v: the three widths are
// multiples of 8). Its filter comes transposed, wt [taps, channels], so that a thread's 8 weights of a tap are 32 contiguous bytes and a
// warp's are one run (read from [channels, taps], every load of a warp touched 32 lines, and the kernel was slower than the scalar one). ROLL: every request brings exactly one token (a decode step), so the thread that filters a channel is the only one
// that reads its tail and rolls it forward itself; otherwise the roll kernel follows.
template <bool ROLL>
__global__ void conv_qkv_store_bf16x8_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ v_out, const __nv_bfloat16* __restrict__ proj, int n_tokens, int proj_stride,
    int cq, int ck, int cv, int taps, const float* __restrict__ wt, const float* __restrict__ bias, float* __restrict__ tails, long long slot_stride,
    const int* __restrict__ req_of_token, const int* __restrict__ cu_q, const int* __restrict__ state_slots, const int* __restrict__ positions,
    float temp_coef, int temp_every, const float* __restrict__ blend, const __nv_bfloat16* __restrict__ first, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ slots, long long n_slots, int* status, const HeadWidths hw) {
    // a block: 8 neighbouring tokens (one per warp) x 256 channels (8 per lane), so that the rows a token shares with its neighbours
    // come out of this SM's L1
    const int c = (blockIdx.y * 32 + (threadIdx.x & 31)) * 8;
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int channels = cq + ck + cv;
    if (c >= channels || t >= n_tokens) return;
    const int r = ROLL ? t : req_of_token[t];
    const int i = ROLL ? 0 : t - cu_q[r];
    float b[8], acc[8], cur[8], wj[8];
    auto load8f = [&](const float* src, float* out) {      // 8 floats from a 32-byte aligned run
        const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
        out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
        out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
    };
    if (bias != nullptr) load8f(bias + c, b);
    else
#pragma unroll
        for (int k = 0; k < 8; ++k) b[k] = 0.f;
    auto load8 = [&](int row, float* out) {
        const Bf16x8 raw = *reinterpret_cast<const Bf16x8*>(proj + (size_t)row * proj_stride + c);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(raw.v[k]);
            out[2 * k] = f.x + b[2 * k];
            out[2 * k + 1] = f.y + b[2 * k + 1];
        }
    };
    load8(t, cur);
    float* tail = taps > 1 ? tails + (long long)state_slots[r] * slot_stride + (long long)c * (taps - 1) : nullptr;
    if (taps <= 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = cur[k];
    } else {
        load8f(wt + (size_t)(taps - 1) * channels + c, wj);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = wj[k] * cur[k];
        for (int j = 0; j < taps - 1; ++j) {
            const int back = taps - 1 - j;
            float u[8];
            if (i - back >= 0) {
                load8(t - back, u);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) u[k] = tail[k * (taps - 1) + taps - 1 + (i - back)];
            }
            load8f(wt + (size_t)j * channels + c, wj);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = fmaf(wj[k], u[k], acc[k]);
        }
        if (ROLL && taps > 1) {
            for (int k = 0; k < 8; ++k) {
                float* tk = tail + k * (taps - 1);
                for (int e = 0; e + 1 < taps - 1; ++e) tk[e] = tk[e + 1];
                tk[taps - 2] = cur[k];
            }
        }
    }
    conv_finish8(acc, c, t, q_out, v_out, cq, ck, cv, positions, temp_coef, temp_every, blend, first, k_pool, v_pool, slots, n_slots, status, hw);
}

// Portions of prompts, filters of 2 to 4 taps: a warp walks over TOK neighbouring tokens and keeps the filter's weights and the last
// TAPS-1 rows in registers, so every row is read once (and TAPS-1 rows before the warp's first token), the weights once a warp.
// Whether a row belongs to the token's own request is decided tap by tap (a row of the packed step before the request's first token
// of this step is another request's: the request's tail stands in for it).
template <int TAPS, int TOK>
__global__ void __launch_bounds__(256) conv_qkv_store_bf16x8_window_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ v_out, const __nv_bfloat16* __restrict__ proj, int n_tokens, int proj_stride,
    int cq, int ck, int cv, const float* __restrict__ wt, const float* __restrict__ bias, const float* __restrict__ tails, long long slot_stride,
    const int* __restrict__ req_of_token, const int* __restrict__ cu_q, const int* __restrict__ state_slots, const int* __restrict__ positions,
    float temp_coef, int temp_every, const float* __restrict__ blend, const __nv_bfloat16* __restrict__ first, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ slots, long long n_slots, int* status, const HeadWidths hw) {
    const int c = (blockIdx.y * 32 + (threadIdx.x & 31)) * 8;
    const int t0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * TOK;
    const int channels = cq + ck + cv;
    if (c >= channels || t0 >= n_tokens) return;
    float b[8], w[TAPS][8], win[TAPS - 1][8];
    auto load8f = [&](const float* src, float* out) {
        const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
        out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
        out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
    };
    if (bias != nullptr) load8f(bias + c, b);
    else
#pragma unroll
        for (int k = 0; k < 8; ++k) b[k] = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) load8f(wt + (size_t)j * channels + c, w[j]);
    auto load8 = [&](int row, float* out) {
        const Bf16x8 raw = *reinterpret_cast<const Bf16x8*>(proj + (size_t)row * proj_stride + c);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(raw.v[k]);
            out[2 * k] = f.x + b[2 * k];
            out[2 * k + 1] = f.y + b[2 * k + 1];
        }
    };
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {       // win[j]: the row TAPS-1-j tokens before the current one
        const int row = t0 - (TAPS - 1) + j;
        if (row >= 0) load8(row, win[j]);
        else
#pragma unroll
            for (int k = 0; k < 8; ++k) win[j][k] = 0.f;
    }
    Bf16x8 rows[TOK];      // the warp's own rows, all requested before the first is used
#pragma unroll
    for (int n = 0; n < TOK; ++n)
        if (t0 + n < n_tokens) rows[n] = *reinterpret_cast<const Bf16x8*>(proj + (size_t)(t0 + n) * proj_stride + c);
#pragma unroll
    for (int n = 0; n < TOK; ++n) {
        const int t = t0 + n;
        if (t >= n_tokens) break;
        const int r = req_of_token[t], i = t - cu_q[r];
        const float* tail = tails + (long long)state_slots[r] * slot_stride + (long long)c * (TAPS - 1);
        float cur[8], acc[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(rows[n].v[k]);
            cur[2 * k] = f.x + b[2 * k];
            cur[2 * k + 1] = f.y + b[2 * k + 1];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = w[TAPS - 1][k] * cur[k];
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j) {
            const int back = TAPS - 1 - j;
            if (i - back >= 0) {
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(w[j][k], win[j][k], acc[k]);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(w[j][k], tail[k * (TAPS - 1) + TAPS - 1 + (i - back)], acc[k]);
            }
        }
#pragma unroll
        for (int j = 0; j + 1 < TAPS - 1; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) win[j][k] = win[j + 1][k];
#pragma unroll
        for (int k = 0; k < 8; ++k) win[TAPS - 2][k] = cur[k];
        conv_finish8(acc, c, t, q_out, v_out, cq, ck, cv, positions, temp_coef, temp_every, blend, first, k_pool, v_pool, slots, n_slots, status, hw);
    }
}

// After the convolution read it: the tail becomes the last taps-1 values of (old tail ++ the step's proj + bias).
template <typename T>
__global__ void conv_qkv_roll_kernel(float* __restrict__ tails, long long slot_stride, const T* __restrict__ proj, int proj_stride, int channels,
                                     int taps, const float* __restrict__ bias, const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int r = blockIdx.x;
    if (c >= channels) return;
    const int t0 = cu_q[r], q = cu_q[r + 1] - t0, keep = taps - 1;
    if (q <= 0) return;
    const float b = bias != nullptr ? bias[c] : 0.f;
    float* tail = tails + (long long)state_slots[r] * slot_stride + (long long)c * keep;
    for (int k = 0; k < keep; ++k) {       // entry k reads entry k + q (not yet overwritten) or a new value
        const int src = q + k - keep;
        tail[k] = src >= 0 ? Num<T>::to_f32(proj[(size_t)(t0 + src) * proj_stride + c]) + b : tail[k + q];
    }
}

OXR_API int oxr_conv_qkv_store(void* q_out, void* v_out, const void* proj, int n_tokens, int n_requests, int proj_stride, int cq, int ck, int cv,
                               int taps, const float* w, const float* wt, const float* bias, float* tails, long long slot_stride, const int* req_of_token,
                               const int* cu_q, const int* state_slots, const int* positions, float temp_coef, int temp_every,
                               const float* blend, const void* first, void* k_pool, void* v_pool, const int* slots, long long n_slots, int dtype,
                               int single_tokens, int dk, int dv, int qw, int kw, int vw, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int channels = cq + ck + cv;
    if (dk <= 0 || dv <= 0 || cq % dk || ck % dk || cv % dv || qw < dk || kw < dk || vw < dv) return OXR_BAD_ARGUMENT;
    const HeadWidths hw = {dk, dv, qw, kw, vw};
    if (cq <= 0 || ck <= 0 || cv <= 0 || taps < 0 || proj_stride < channels || n_requests <= 0 || (taps > 0 && w == nullptr) ||
        (taps > 1 && tails == nullptr) || (blend != nullptr && first == nullptr))
        return OXR_BAD_ARGUMENT;
    const int threads = 128;
    dim3 grid(n_tokens, (channels + threads - 1) / threads), roll(n_requests, (channels + threads - 1) / threads);
    if (grid.y > 65535) return OXR_BAD_ARGUMENT;
#define OXR_CONV_QKV(T) \
    do { \
        conv_qkv_store_kernel<T><<<grid, threads, 0, stream>>>((T*)q_out, (T*)v_out, (const T*)proj, proj_stride, cq, ck, cv, taps, w, bias, tails, \
                                                              slot_stride, req_of_token, cu_q, state_slots, positions, temp_coef, temp_every, blend, \
                                                              (const T*)first, (T*)k_pool, (T*)v_pool, slots, n_slots, status, hw); \
        if (taps > 1) \
            conv_qkv_roll_kernel<T><<<roll, threads, 0, stream>>>(tails, slot_stride, (const T*)proj, proj_stride, channels, taps, bias, cu_q, \
                                                                 state_slots); \
    } while (0)
    const auto aligned = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (dtype == 1 && dk % 8 == 0 && dv % 8 == 0 && qw % 8 == 0 && kw % 8 == 0 && vw % 8 == 0 && proj_stride % 8 == 0 && aligned(proj) && aligned(q_out) && aligned(v_out) &&
        aligned(first) && aligned(k_pool) && aligned(v_pool) && (taps == 0 || wt != nullptr) && aligned(wt) && aligned(bias)) {
        using B = __nv_bfloat16;
        dim3 vgrid((n_tokens + 7) / 8, (channels / 8 + 31) / 32);
        const bool single = n_tokens == n_requests && single_tokens;
#define OXR_CONV_QKV8(ROLL) \
        conv_qkv_store_bf16x8_kernel<ROLL><<<vgrid, 256, 0, stream>>>((B*)q_out, (B*)v_out, (const B*)proj, n_tokens, proj_stride, cq, ck, cv, taps, wt, bias, \
                                                                         tails, slot_stride, req_of_token, cu_q, state_slots, positions, temp_coef, \
                                                                         temp_every, blend, (const B*)first, (B*)k_pool, (B*)v_pool, slots, n_slots, status, hw)
#define OXR_CONV_QKV8W(TAPS) \
        conv_qkv_store_bf16x8_window_kernel<TAPS, 8><<<dim3((n_tokens + 63) / 64, (channels / 8 + 31) / 32), 256, 0, stream>>>( \
            (B*)q_out, (B*)v_out, (const B*)proj, n_tokens, proj_stride, cq, ck, cv, wt, bias, tails, slot_stride, req_of_token, cu_q, state_slots, \
            positions, temp_coef, temp_every, blend, (const B*)first, (B*)k_pool, (B*)v_pool, slots, n_slots, status, hw)
        if (single) {
            OXR_CONV_QKV8(true);
        } else {
            if (taps == 2 && n_tokens >= 64) OXR_CONV_QKV8W(2);
            else if (taps == 3 && n_tokens >= 64) OXR_CONV_QKV8W(3);
            else if (taps == 4 && n_tokens >= 64) OXR_CONV_QKV8W(4);
            else OXR_CONV_QKV8(false);
            if (taps > 1)
                conv_qkv_roll_kernel<B><<<roll, threads, 0, stream>>>(tails, slot_stride, (const B*)proj, proj_stride, channels, taps, bias, cu_q, state_slots);
        }
#undef OXR_CONV_QKV8W
#undef OXR_CONV_QKV8
        return oxr_launch_status();
    }
    if (dtype == 0) OXR_CONV_QKV(float);
    else OXR_CONV_QKV(__nv_bfloat16);
#undef OXR_CONV_QKV
    return oxr_launch_status();
}

// x[t, c] += row[c] in place, the sum in fp32
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ row, size_t total, int width) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = Num<T>::from_f32(Num<T>::to_f32(x[i]) + row[i % width]);
}

OXR_API int oxr_add_bias(void* x, const float* row, int n, int width, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n * width;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, row, total, width);
    else add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)x, row, total, width);
    return oxr_launch_status();
}

__global__ void scale_f32_kernel(float* __restrict__ x, float scale, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] *= scale;
}

OXR_API int oxr_scale_f32(float* x, float scale, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    scale_f32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, scale, (size_t)total);
    return oxr_launch_status();
}
