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

template <typename T>
__global__ void conv_qkv_store_kernel(
    T* __restrict__ q_out, T* __restrict__ v_out, const T* __restrict__ proj, int proj_stride, int cq, int ck, int cv, int taps,
    const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ tails, long long slot_stride,
    const int* __restrict__ req_of_token, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
    const int* __restrict__ positions, float temp_coef, int temp_every, const float* __restrict__ blend, const T* __restrict__ first,
    T* __restrict__ k_pool, T* __restrict__ v_pool, const int* __restrict__ slots, long long n_slots, int* status) {
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
        q_out[(size_t)t * cq + c] = Num<T>::from_f32(acc);
        return;
    }
    const long long slot = slots[t];
    if (slot >= n_slots) oxr_report(status, OXR_BAD_SLOT, t);
    const bool store = slot >= 0 && slot < n_slots;
    if (c < cq + ck) {
        if (store) k_pool[slot * ck + (c - cq)] = Num<T>::from_f32(acc);
        return;
    }
    const int cc = c - cq - ck;
    if (blend != nullptr) {
        const float lam = blend[0];
        acc = (1.f - lam) * acc + lam * Num<T>::to_f32(first[(size_t)t * cv + cc]);
    }
    const T rounded = Num<T>::from_f32(acc);
    if (v_out != nullptr) v_out[(size_t)t * cv + cc] = rounded;
    if (store) v_pool[slot * cv + cc] = rounded;
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
                               int taps, const float* w, const float* bias, float* tails, long long slot_stride, const int* req_of_token,
                               const int* cu_q, const int* state_slots, const int* positions, float temp_coef, int temp_every,
                               const float* blend, const void* first, void* k_pool, void* v_pool, const int* slots, long long n_slots, int dtype,
                               int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int channels = cq + ck + cv;
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
                                                              (const T*)first, (T*)k_pool, (T*)v_pool, slots, n_slots, status); \
        if (taps > 1) \
            conv_qkv_roll_kernel<T><<<roll, threads, 0, stream>>>(tails, slot_stride, (const T*)proj, proj_stride, channels, taps, bias, cu_q, \
                                                                 state_slots); \
    } while (0)
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
